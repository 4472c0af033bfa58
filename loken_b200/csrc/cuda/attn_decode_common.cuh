// Shared tail of the flash-decode kernels: merge the four warps' running (max, sum, out),
// merge the key splits (the block that arrives last on the (row, kv head) counter does it),
// add the attention sink, normalise and write bf16 or e4m3 + per-head scale.
#pragma once
#include "common.cuh"
#include "tc100.cuh"

namespace lk {

struct DecodeParamsV2 {
  const __nv_bfloat16* q;   // [rows, n_q, hd]
  const __half* k_scale;    // [slots, n_kv, hd/32]
  const __half* v_scale;
  const int* block_table;
  const int* row_seq;
  const int* seq_lens;
  const float* sinks;
  __nv_bfloat16* out;
  uint8_t* out_fp8;
  float* out_scales_t;
  long long scale_ld;
  float* ws;
  int* counters;
  int* status;
  long long num_slots;
  int n_q, n_kv, max_blocks, block_size, window;
  float scale_log2;
};

// sm_m / sm_l: [NW][G]; sm_o: [NW][G][HD] (NW partial results, one per warp in the SIMT kernels);
// every thread of the 128 finishing threads calls this.
template <int HD, int G, int NW = 4>
__device__ __forceinline__ void decode_finish(const DecodeParamsV2& p, int row, int kvh, int split, int nsplit,
                                              const float (*sm_m)[G], const float (*sm_l)[G],
                                              const float (*sm_o)[G][HD], int* s_last, float* red, int d) {
  constexpr float LOG2E = 1.4426950408889634f;
  const int row_kv = row * p.n_kv + kvh;
  float fm[G], fl[G], fo[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float mm = sm_m[0][g];
#pragma unroll
    for (int w = 1; w < NW; ++w) mm = fmaxf(mm, sm_m[w][g]);
    float ll = 0.f, oo = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const float a = (sm_m[w][g] > -INFINITY) ? exp2f(sm_m[w][g] - mm) : 0.f;
      ll += sm_l[w][g] * a;
      if (d < HD) oo += sm_o[w][g][d] * a;
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
    // one thread's fences order the partial before the counter and the counter before the merge
    asm volatile("bar.sync 2, 128;" ::: "memory");
    if (d == 0) {
      __threadfence();
      const int prev = atomicAdd(&p.counters[row_kv], 1);
      *s_last = (prev == nsplit - 1);
      if (*s_last) p.counters[row_kv] = 0;
      __threadfence();
    }
    asm volatile("bar.sync 2, 128;" ::: "memory");
    if (!*s_last) return;
    // One pass over the splits with a running (max, sum, out): every split costs one round trip
    // to memory (its 3 G values are independent loads), not one per head and quantity.
    const float* all = p.ws + (long long)row_kv * nsplit * (G * (HD + 2));
#pragma unroll
    for (int g = 0; g < G; ++g) {
      fm[g] = -INFINITY;
      fl[g] = 0.f;
      fo[g] = 0.f;
    }
    for (int s = 0; s < nsplit; ++s) {
      float ms[G], ls[G], os[G];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float* base = all + (s * G + g) * (HD + 2);
        ms[g] = __ldcg(base + HD);
        ls[g] = __ldcg(base + HD + 1);
        os[g] = d < HD ? __ldcg(base + d) : 0.f;
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float mn = fmaxf(fm[g], ms[g]);
        const float a0 = (fm[g] > -INFINITY) ? exp2f(fm[g] - mn) : 0.f;
        const float a1 = (ms[g] > -INFINITY) ? exp2f(ms[g] - mn) : 0.f;
        fl[g] = fl[g] * a0 + ls[g] * a1;
        fo[g] = fo[g] * a0 + os[g] * a1;
        fm[g] = mn;
      }
    }
  }
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
      // hd == 128: one head is one 128-group of the o_proj input.  Block max over 128 threads.
      const float r = bf2f(f2bf(d < HD ? val : 0.f));
      float a = warp_max(fabsf(r));
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if ((d & 31) == 0) red[d >> 5] = a;
      asm volatile("bar.sync 2, 128;" ::: "memory");
      const float amax = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
      const float sc = e4m3_group_scale(amax);
      if (d < HD) p.out_fp8[(long long)row * p.n_q * HD + head * HD + d] = f2e4m3(r / sc);
      if (d == 0) p.out_scales_t[(long long)head * p.scale_ld + row] = sc;
    }
  }
}

}  // namespace lk
