// Token sampling on the device, one block per row of [B, vocab] fp32 logits.
//
//   lk_argmax          greedy: first maximum wins (lowest index on ties)
//   lk_repeat_penalty  positive logit / penalty, negative logit * penalty, once per distinct
//                      token of the row's recent window
//   lk_sample          temperature, min-p floor, top-k, then nucleus (top-p measured against
//                      the mass that survived top-k), then one draw with a host-supplied
//                      uniform u in [0, 1).  T < 1e-7 means greedy.
//
// Nothing is sorted.  Top-k is a 4-pass radix select over an order-preserving integer key of
// the logit; the nucleus cut is the same descent with probability mass per bin instead of a
// count.  Mass is carried in 2^-40 fixed point (u64), so bin sums do not depend on the order
// in which threads add and a (logits, u) pair always yields the same token.  Ties at a cut
// are resolved by index.  The draw walks the surviving tokens in index order, which gives the
// same distribution as walking them by probability.
//
// Counterparts in the reference: cuda/sampling.cu (batched argmax, top-k + denominator,
// repeat penalty), sample_topk_block_f32 / sample_topk_final_f32 in src/inference/cuda/fused.cu,
// and the host semantics in src/inference/sample/token_sampling.rs.
#include <cooperative_groups.h>

#include "common.cuh"
#include "host_common.h"
#include "loken_cuda.h"

using namespace lk;

namespace {

constexpr int NT = 1024;
typedef unsigned long long u64;

__device__ __forceinline__ uint32_t fkey(float x) {
  uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// 64-bit bin += v on two 32-bit words (adds commute, so the result does not depend on thread order)
__device__ __forceinline__ void hist_add(uint32_t* lo, uint32_t* hi, int b, u64 v) {
  const uint32_t vl = (uint32_t)v, vh = (uint32_t)(v >> 32);
  const uint32_t old = atomicAdd(&lo[b], vl);
  const uint32_t carry = (old + vl < old) ? 1u : 0u;
  if (vh + carry) atomicAdd(&hi[b], vh + carry);
}
__device__ __forceinline__ u64 hist_get(const uint32_t* lo, const uint32_t* hi, int b) {
  return ((u64)hi[b] << 32) | (u64)lo[b];
}

__device__ __forceinline__ u64 block_sum_u64(u64 v, u64* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  u64 t = (lane < (NT >> 5)) ? red[lane] : 0ull;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

// Exclusive prefix of per-thread values in thread order; returns the prefix and the total.
__device__ __forceinline__ u64 block_excl_scan_u64(u64 v, u64* red, u64* total) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  u64 inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    u64 t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  __syncthreads();
  if (lane == 31) red[w] = inc;
  __syncthreads();
  if (w == 0) {
    u64 x = red[lane];
    u64 xi = x;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      u64 t = __shfl_up_sync(0xffffffffu, xi, o);
      if (lane >= o) xi += t;
    }
    red[lane] = xi - x;       // exclusive warp offsets
    if (lane == 31) red[32] = xi;
  }
  __syncthreads();
  *total = red[32];
  return red[w] + inc - v;
}

// Smallest index i with sum_{j <= i} f(j) >= target (target >= 1), walking the row in index order
// with coalesced reads: each warp owns one contiguous slice, slices' totals are scanned, and the
// one warp whose slice holds the crossing walks it again 32 values at a time.  Returns
// 0x7fffffff when the whole row sums to less than the target.  Called by the whole block.
template <class F>
__device__ __forceinline__ int ordered_find(int V, F f, u64 target, u64* red, int* s_out, u64* total_out) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int per = (((V + 31) / 32) + 31) & ~31;
  const int b0 = min(V, w * per), b1 = min(V, b0 + per);
  u64 part = 0;
  for (int i = b0 + lane; i < b1; i += 32) part += f(i);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  __syncthreads();
  if (lane == 0) red[w] = part;
  if (threadIdx.x == 0) *s_out = 0x7fffffff;
  __syncthreads();
  const u64 x = red[lane];
  u64 inc = x;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const u64 t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  const u64 total = __shfl_sync(0xffffffffu, inc, 31);
  const u64 before_w = __shfl_sync(0xffffffffu, inc - x, w);
  const u64 mine_w = __shfl_sync(0xffffffffu, x, w);
  if (before_w < target && before_w + mine_w >= target) {
    u64 run = before_w;
    for (int base = b0; base < b1; base += 32) {
      const int i = base + lane;
      const u64 v = i < b1 ? f(i) : 0ull;
      u64 s = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const u64 t = __shfl_up_sync(0xffffffffu, s, o);
        if (lane >= o) s += t;
      }
      const unsigned hit = __ballot_sync(0xffffffffu, run + s >= target);
      if (hit) {
        if (lane == __ffs(hit) - 1) *s_out = i;
        break;
      }
      run += __shfl_sync(0xffffffffu, s, 31);
    }
  }
  __syncthreads();
  *total_out = total;
  return *s_out;
}

struct RowCtx {
  const float* x;
  int V;
  float mx, invT, floor_x;
};

__device__ __forceinline__ u64 mass_of(const RowCtx& c, float xv) {
  // exp((x - max) / T) in 2^-40 fixed point; a token whose weight underflows (a masked
  // logit of -inf among them) carries no mass and can never be drawn
  const float w = __expf((xv - c.mx) * c.invT);
  return (u64)(w * 1099511627776.0f);
}

// Set membership: a lower key bound (exclusive) with ties admitted up to an index.
struct Cut {
  uint32_t key;     // keys above this are in
  int tie_last;     // keys equal to this are in when index <= tie_last
};
__device__ __forceinline__ bool in_cut(const Cut& c, uint32_t k, int i) {
  return k > c.key || (k == c.key && i <= c.tie_last);
}

__global__ void __launch_bounds__(NT)
argmax_kernel(const float* __restrict__ logits, long long ld, int V, int* __restrict__ out) {
  __shared__ float smax[32];
  __shared__ int sidx[32];
  const float* x = logits + (long long)blockIdx.x * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += NT) {
    const float v = x[i];
    if (v > best || (v == best && i < bi)) {
      best = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) {
    smax[w] = best;
    sidx[w] = bi;
  }
  __syncthreads();
  if (w == 0) {
    best = smax[lane];
    bi = sidx[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    if (lane == 0) out[blockIdx.x] = (bi == 0x7fffffff) ? 0 : bi;
  }
}

__global__ void repeat_penalty_kernel(float* __restrict__ logits, long long ld, int V, const int* __restrict__ recent,
                                      int L, const float* __restrict__ penalty) {
  const int row = blockIdx.x;
  const float pen = penalty[row];
  if (pen == 1.f) return;
  const int* r = recent + (long long)row * L;
  float* x = logits + (long long)row * ld;
  for (int i = threadIdx.x; i < L; i += blockDim.x) {
    const int t = r[i];
    if (t < 0 || t >= V) continue;   // padding or a bad id: skip, never index outside the row
    bool dup = false;
    for (int j = 0; j < i; ++j) dup |= (r[j] == t);
    if (dup) continue;
    const float v = x[t];
    x[t] = v > 0.f ? v / pen : v * pen;
  }
}

// Per-row token rules ahead of the sampler: up to R (id, value) pairs per row.  mode 0 adds the
// value to the logit (a ban is a value of -inf); mode 1 keeps only the listed ids (their values
// are added) and sets every other logit to -inf.  Ids outside [0, V) are skipped.
constexpr int RULES_MAX = 512;
__global__ void token_rules_kernel(float* __restrict__ logits, long long ld, int V, const int* __restrict__ ids,
                                   const float* __restrict__ vals, const int* __restrict__ counts,
                                   const int* __restrict__ modes, int R) {
  __shared__ float kept[RULES_MAX];
  const int row = blockIdx.x;
  const int n = min(counts[row], min(R, RULES_MAX));
  const int mode = modes[row];
  if (n <= 0 && mode == 0) return;
  float* x = logits + (long long)row * ld;
  const int* id = ids + (long long)row * R;
  const float* vl = vals + (long long)row * R;
  if (mode == 0) {
    // a repeated id takes each of its values once: one thread per entry, atomics not needed
    // because an id is applied by the first entry that names it with the sum of all of them
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const int t = id[i];
      if (t < 0 || t >= V) continue;
      bool first = true;
      float sum = 0.f;
      for (int j = 0; j < n; ++j)
        if (id[j] == t) { if (j < i) first = false; sum += vl[j]; }
      if (first) x[t] += sum;
    }
    return;
  }
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int t = id[i];
    kept[i] = (t >= 0 && t < V) ? x[t] + vl[i] : 0.f;
  }
  __syncthreads();
  const float ninf = __int_as_float(0xff800000);
  for (int j = threadIdx.x; j < V; j += blockDim.x) x[j] = ninf;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int t = id[i];
    if (t >= 0 && t < V) x[t] = kept[i];
  }
}

// Grammar masks: bit t of row r's mask words says token t may be sampled; the rest become -inf.
// rows with has[r] == 0 are left alone.
__global__ void token_bitmask_kernel(float* __restrict__ logits, long long ld, int V,
                                     const uint32_t* __restrict__ bits, int words, const int* __restrict__ has) {
  const int row = blockIdx.y;
  if (has && !has[row]) return;
  const uint32_t* m = bits + (long long)row * words;
  float* x = logits + (long long)row * ld;
  const float ninf = __int_as_float(0xff800000);
  for (int w = blockIdx.x * blockDim.x + threadIdx.x; w < words; w += gridDim.x * blockDim.x) {
    const uint32_t b = m[w];
    if (b == 0xffffffffu) continue;
    const int t0 = w * 32;
#pragma unroll 8
    for (int i = 0; i < 32; ++i)
      if (!((b >> i) & 1u) && t0 + i < V) x[t0 + i] = ninf;
  }
}

__global__ void __launch_bounds__(NT)
sample_kernel(const float* __restrict__ logits, long long ld, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
              const float* __restrict__ uniform, int* __restrict__ out) {
  // bins as two 32-bit words: native shared-memory adds with a carry, instead of 64-bit
  // compare-and-swap loops that serialise when many threads meet in one bin
  __shared__ uint32_t hist_lo[256], hist_hi[256];
  __shared__ u64 red[33];
  __shared__ float fred[32];
  __shared__ uint32_t s_prefix;
  __shared__ u64 s_acc;        // count or mass of the bins above the chosen one
  __shared__ int s_int;

  const int row = blockIdx.x;
  RowCtx c;
  c.x = logits + (long long)row * ld;
  c.V = V;
  const float T = temperature[row];

  // row maximum (and greedy exit)
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += NT) {
    const float v = c.x[i];
    if (v > best || (v == best && i < bi)) {
      best = v;
      bi = i;
    }
  }
  c.mx = block_max(best, fred);
  if (T < 1e-7f) {
    // lowest index among the maxima
    int cand = (best == c.mx) ? bi : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) fred[threadIdx.x >> 5] = __int_as_float(cand);
    __syncthreads();
    if (threadIdx.x < 32) {
      int v = __float_as_int(fred[threadIdx.x]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, o));
      if (threadIdx.x == 0) out[row] = (v == 0x7fffffff) ? 0 : v;
    }
    return;
  }
  c.invT = 1.f / T;
  const float mp = min_p ? min_p[row] : 0.f;
  c.floor_x = (mp > 0.f) ? c.mx + __logf(mp) * T : -INFINITY;
  const uint32_t floor_key = (mp > 0.f) ? fkey(c.floor_x) : 0u;
  const int k = top_k ? top_k[row] : 0;
  const float tp = top_p ? top_p[row] : 1.f;

  // contiguous chunk of this thread for the index-ordered passes
  const int C = (V + NT - 1) / NT;
  const int c0 = min(V, threadIdx.x * C), c1 = min(V, c0 + C);

  // ---------------- top-k: radix select by count among the keys at or above the floor ----------
  Cut cut_k;
  cut_k.key = 0u;
  cut_k.tie_last = 0x7fffffff;
  if (k > 0 && k < V) {
    uint32_t prefix = 0, mask = 0;
    u64 above = 0;
    for (int shift = 24; shift >= 0; shift -= 8) {
      for (int b = threadIdx.x; b < 256; b += NT) { hist_lo[b] = 0; hist_hi[b] = 0; }
      __syncthreads();
      {
        // neighbouring logits mostly share their leading key bits: runs of equal bins are summed
        // in a register and flushed once, which keeps the shared-memory atomics from serialising
        int run_bin = -1;
        u64 run = 0;
        for (int i = threadIdx.x; i < V; i += NT) {
          const uint32_t kk = fkey(c.x[i]);
          if (kk >= floor_key && (kk & mask) == prefix) {
            const int b = (kk >> shift) & 255u;
            if (b != run_bin) {
              if (run) hist_add(hist_lo, hist_hi, run_bin, run);
              run_bin = b;
              run = 0;
            }
            ++run;
          }
        }
        if (run) hist_add(hist_lo, hist_hi, run_bin, run);
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        u64 acc = above;
        int b = 255;
        for (; b > 0; --b) {
          if (acc + hist_get(hist_lo, hist_hi, b) >= (u64)k) break;
          acc += hist_get(hist_lo, hist_hi, b);
        }
        s_prefix = prefix | ((uint32_t)b << shift);
        s_acc = acc;
      }
      __syncthreads();
      prefix = s_prefix;
      above = s_acc;
      mask |= 255u << shift;
      __syncthreads();
    }
    // prefix = key of the k-th largest; `above` keys are larger; admit `need` of the equal ones by index
    const u64 need = (u64)k > above ? (u64)k - above : 0ull;
    u64 total;
    int tie = -1;
    if (need > 0)
      tie = ordered_find(V, [&](int i) -> u64 { return fkey(c.x[i]) == prefix ? 1ull : 0ull; }, need, red, &s_int,
                         &total);
    cut_k.key = prefix;
    cut_k.tie_last = tie;
  }
#define IN_K(kk, i) ((kk) >= floor_key && in_cut(cut_k, (kk), (i)))

  // ---------------- nucleus: radix descent by mass inside the top-k set ----------------
  Cut cut_p;
  cut_p.key = 0u;
  cut_p.tie_last = 0x7fffffff;
  if (tp < 1.f) {
    u64 zk = 0;
    for (int i = threadIdx.x; i < V; i += NT) {
      const float xv = c.x[i];
      const uint32_t kk = fkey(xv);
      if (IN_K(kk, i)) zk += mass_of(c, xv);
    }
    zk = block_sum_u64(zk, red);
    u64 target = (u64)((double)zk * (double)tp);
    if (target < 1) target = 1;
    uint32_t prefix = 0, mask = 0;
    u64 above = 0;
    for (int shift = 24; shift >= 0; shift -= 8) {
      for (int b = threadIdx.x; b < 256; b += NT) { hist_lo[b] = 0; hist_hi[b] = 0; }
      __syncthreads();
      {
        int run_bin = -1;
        u64 run = 0;
        for (int i = threadIdx.x; i < V; i += NT) {
          const float xv = c.x[i];
          const uint32_t kk = fkey(xv);
          if ((kk & mask) == prefix && IN_K(kk, i)) {
            const int b = (kk >> shift) & 255u;
            if (b != run_bin) {
              if (run) hist_add(hist_lo, hist_hi, run_bin, run);
              run_bin = b;
              run = 0;
            }
            run += mass_of(c, xv);
          }
        }
        if (run) hist_add(hist_lo, hist_hi, run_bin, run);
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        u64 acc = above;
        int b = 255;
        for (; b > 0; --b) {
          if (acc + hist_get(hist_lo, hist_hi, b) >= target) break;
          acc += hist_get(hist_lo, hist_hi, b);
        }
        s_prefix = prefix | ((uint32_t)b << shift);
        s_acc = acc;
      }
      __syncthreads();
      prefix = s_prefix;
      above = s_acc;
      mask |= 255u << shift;
      __syncthreads();
    }
    // tokens with key == prefix are admitted in index order until the running mass reaches
    // the target: the token that crosses p is kept
    const u64 need = target > above ? target - above : 1ull;
    u64 total;
    const int tie = ordered_find(V, [&](int i) -> u64 {
      const float xv = c.x[i];
      const uint32_t kk = fkey(xv);
      return (kk == prefix && IN_K(kk, i)) ? mass_of(c, xv) : 0ull;
    }, need, red, &s_int, &total);
    cut_p.key = prefix;
    cut_p.tie_last = tie;
  }

  // ---------------- draw ----------------
  auto final_mass = [&](int i) -> u64 {
    const float xv = c.x[i];
    const uint32_t kk = fkey(xv);
    return (IN_K(kk, i) && in_cut(cut_p, kk, i)) ? mass_of(c, xv) : 0ull;
  };
  u64 zsum = 0;
  for (int i = threadIdx.x; i < V; i += NT) zsum += final_mass(i);
  zsum = block_sum_u64(zsum, red);
  float u = uniform[row];
  u = fminf(fmaxf(u, 0.f), 0.99999994f);
  u64 r = (u64)((double)zsum * (double)u);
  if (r >= zsum) r = zsum ? zsum - 1 : 0;
  u64 total;
  int drawn = zsum ? ordered_find(V, final_mass, r + 1, red, &s_int, &total) : -1;
  if (drawn == 0x7fffffff) drawn = -1;
#undef IN_K
  if (threadIdx.x == 0) {
    int tok = drawn;
    if (tok < 0) {
      // an empty set (a row without a finite value): fall back to the first maximum
      tok = 0;
      float bv = -INFINITY;
      for (int i = 0; i < V; ++i)
        if (c.x[i] > bv) {
          bv = c.x[i];
          tok = i;
        }
    }
    out[row] = tok;
  }
}

// ---- the same sampler on a thread-block cluster ------------------------------------------------------
// One CTA walks a row of 128k logits a dozen times (row maximum, four radix passes per cut, the mass sums,
// the index-ordered searches): 0.3 ms per step whatever the batch, a tenth of a single-stream step.  Here
// eight CTAs of a cluster share a row.  A thread keeps VPT consecutive logits in registers for the whole
// kernel, so the row is read from memory once; histograms are built per CTA and merged through distributed
// shared memory (every CTA reads the eight copies and comes to the same cut); sums and the index-ordered
// searches go through one word per CTA.  Masses are the same 2^-40 fixed-point integers, so every sum, cut
// and draw equals the one-CTA kernel's bit for bit.  Buffers that other CTAs read alternate between two
// copies: a copy is rewritten two exchanges later, after a cluster barrier that no CTA passes before every
// reader of the old contents is done.
namespace cg = cooperative_groups;
constexpr int CS = 8;           // CTAs per row

struct ClusterShared {
  uint32_t hist_lo[2][256], hist_hi[2][256];
  u64 merged[256];
  u64 tot[2];
  int res[2];
  u64 red[33];
  float fred[32];
  uint32_t s_prefix;
  u64 s_acc;
};

struct Cl {
  cg::cluster_group cluster;
  ClusterShared* sh;
  int ph, rank;

  __device__ __forceinline__ u64 remote_tot(int r) { return *cluster.map_shared_rank(&sh->tot[ph], r); }

  // sum over the cluster of a per-thread value
  __device__ __forceinline__ u64 sum(u64 v) {
    const u64 t = block_sum_u64(v, sh->red);
    if (threadIdx.x == 0) sh->tot[ph] = t;
    cluster.sync();
    u64 s = 0;
#pragma unroll
    for (int r = 0; r < CS; ++r) s += remote_tot(r);
    ph ^= 1;
    return s;
  }
  // min over the cluster of a per-CTA value every thread of the CTA holds
  __device__ __forceinline__ u64 min_of(u64 mine) {
    if (threadIdx.x == 0) sh->tot[ph] = mine;
    cluster.sync();
    u64 s = ~0ull;
#pragma unroll
    for (int r = 0; r < CS; ++r) s = min(s, remote_tot(r));
    ph ^= 1;
    return s;
  }

  // One radix step.  f(j, &amount) gives the bin of this thread's element j (or -1) and what it adds.
  // Walks the merged bins from the top: the bin in which `above` + bins reaches `target` becomes the next
  // byte of `prefix`; `above` grows by the bins passed.
  template <int VPT, class F>
  __device__ __forceinline__ void radix_step(int nv, F f, u64 target, int shift, uint32_t& prefix, u64& above) {
    uint32_t* lo = sh->hist_lo[ph];
    uint32_t* hi = sh->hist_hi[ph];
    for (int b = threadIdx.x; b < 256; b += NT) {
      lo[b] = 0;
      hi[b] = 0;
    }
    __syncthreads();
    int run_bin = -1;
    u64 run = 0;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      u64 amount = 0;
      const int b = j < nv ? f(j, amount) : -1;
      if (b >= 0) {
        if (b != run_bin) {
          if (run) hist_add(lo, hi, run_bin, run);
          run_bin = b;
          run = 0;
        }
        run += amount;
      }
    }
    if (run) hist_add(lo, hi, run_bin, run);
    cluster.sync();
    if (threadIdx.x < 256) {
      u64 t = 0;
#pragma unroll
      for (int r = 0; r < CS; ++r) {
        const uint32_t l = *cluster.map_shared_rank(&lo[threadIdx.x], r);
        const uint32_t h = *cluster.map_shared_rank(&hi[threadIdx.x], r);
        t += ((u64)h << 32) | (u64)l;
      }
      sh->merged[threadIdx.x] = t;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      u64 acc = above;
      int b = 255;
      for (; b > 0; --b) {
        if (acc + sh->merged[b] >= target) break;
        acc += sh->merged[b];
      }
      sh->s_prefix = prefix | ((uint32_t)b << shift);
      sh->s_acc = acc;
    }
    __syncthreads();
    prefix = sh->s_prefix;
    above = sh->s_acc;
    __syncthreads();
    ph ^= 1;
  }

  // Smallest index of the row at which the running sum of f, in index order, reaches `target` (>= 1);
  // 0x7fffffff when the row sums to less.  f(j) is the amount of this thread's element j; i0 its first index.
  template <int VPT, class F>
  __device__ __forceinline__ int find(int nv, int i0, F f, u64 target, u64* total_out) {
    u64 mine = 0;
#pragma unroll
    for (int j = 0; j < VPT; ++j)
      if (j < nv) mine += f(j);
    u64 btotal;
    const u64 excl = block_excl_scan_u64(mine, sh->red, &btotal);
    if (threadIdx.x == 0) {
      sh->tot[ph] = btotal;
      sh->res[ph] = 0x7fffffff;
    }
    cluster.sync();
    u64 before = 0, total = 0;
#pragma unroll
    for (int r = 0; r < CS; ++r) {
      const u64 t = remote_tot(r);
      if (r < rank) before += t;
      total += t;
    }
    const u64 lo = before + excl;
    if (mine > 0 && lo < target && lo + mine >= target) {        // one thread of the cluster
      u64 run = lo;
      int hit = -1;
#pragma unroll
      for (int j = 0; j < VPT; ++j)
        if (j < nv) {
          run += f(j);
          if (hit < 0 && run >= target) hit = j;
        }
#pragma unroll
      for (int r = 0; r < CS; ++r) *cluster.map_shared_rank(&sh->res[ph], r) = i0 + hit;
    }
    cluster.sync();
    const int out = sh->res[ph];
    ph ^= 1;
    *total_out = total;
    return out;
  }
};

template <int VPT>
__global__ void __launch_bounds__(NT)
sample_cluster_kernel(const float* __restrict__ logits, long long ld, int V, const float* __restrict__ temperature,
                      const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
                      const float* __restrict__ uniform, int* __restrict__ out) {
  __shared__ ClusterShared shared;
  Cl cl{cg::this_cluster(), &shared, 0, 0};
  cl.rank = (int)cl.cluster.block_rank();
  const int row = blockIdx.y;
  RowCtx c;
  c.x = logits + (long long)row * ld;
  c.V = V;
  const float T = temperature[row];

  // this thread's run of the row, kept in registers from here on
  const int i0 = (cl.rank * NT + (int)threadIdx.x) * VPT;
  const int nv = max(0, min(VPT, V - i0));
  float x[VPT];
#pragma unroll
  for (int j = 0; j < VPT; ++j) x[j] = j < nv ? __ldg(c.x + i0 + j) : -INFINITY;

  float best = -INFINITY;
  int bi = 0x7fffffff;
#pragma unroll
  for (int j = 0; j < VPT; ++j)
    if (j < nv && x[j] > best) {
      best = x[j];
      bi = i0 + j;
    }
  {
    // maximum of the row: keys order like the floats, and a minimum of inverted keys travels as an integer
    const float bm = block_max(best, shared.fred);
    c.mx = __uint_as_float(0u);
    const u64 k = cl.min_of((u64)(~fkey(bm)));
    const uint32_t key = ~(uint32_t)k;
    c.mx = __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
  }
  if (T < 1e-7f) {
    // lowest index among the maxima
    int cand = (best == c.mx) ? bi : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) shared.fred[threadIdx.x >> 5] = __int_as_float(cand);
    __syncthreads();
    int v = __float_as_int(shared.fred[threadIdx.x & 31]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, o));
    const u64 all = cl.min_of((u64)(uint32_t)v);
    if (cl.rank == 0 && threadIdx.x == 0) out[row] = (all >= 0x7fffffffull) ? 0 : (int)all;
    cl.cluster.sync();          // no CTA leaves while another may still read its shared memory
    return;
  }
  c.invT = 1.f / T;
  const float mp = min_p ? min_p[row] : 0.f;
  c.floor_x = (mp > 0.f) ? c.mx + __logf(mp) * T : -INFINITY;
  const uint32_t floor_key = (mp > 0.f) ? fkey(c.floor_x) : 0u;
  const int k = top_k ? top_k[row] : 0;
  const float tp = top_p ? top_p[row] : 1.f;

  // ---------------- top-k: radix select by count among the keys at or above the floor ----------
  Cut cut_k;
  cut_k.key = 0u;
  cut_k.tie_last = 0x7fffffff;
  if (k > 0 && k < V) {
    uint32_t prefix = 0, mask = 0;
    u64 above = 0;
    for (int shift = 24; shift >= 0; shift -= 8) {
      cl.template radix_step<VPT>(nv, [&](int j, u64& amount) -> int {
        const uint32_t kk = fkey(x[j]);
        amount = 1;
        return (kk >= floor_key && (kk & mask) == prefix) ? (int)((kk >> shift) & 255u) : -1;
      }, (u64)k, shift, prefix, above);
      mask |= 255u << shift;
    }
    const u64 need = (u64)k > above ? (u64)k - above : 0ull;
    u64 total;
    int tie = -1;
    if (need > 0)
      tie = cl.template find<VPT>(nv, i0, [&](int j) -> u64 { return fkey(x[j]) == prefix ? 1ull : 0ull; }, need, &total);
    cut_k.key = prefix;
    cut_k.tie_last = tie;
  }
#define IN_K(kk, i) ((kk) >= floor_key && in_cut(cut_k, (kk), (i)))

  // ---------------- nucleus: radix descent by mass inside the top-k set ----------------
  Cut cut_p;
  cut_p.key = 0u;
  cut_p.tie_last = 0x7fffffff;
  if (tp < 1.f) {
    u64 zk = 0;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const uint32_t kk = fkey(x[j]);
      if (j < nv && IN_K(kk, i0 + j)) zk += mass_of(c, x[j]);
    }
    zk = cl.sum(zk);
    u64 target = (u64)((double)zk * (double)tp);
    if (target < 1) target = 1;
    uint32_t prefix = 0, mask = 0;
    u64 above = 0;
    for (int shift = 24; shift >= 0; shift -= 8) {
      cl.template radix_step<VPT>(nv, [&](int j, u64& amount) -> int {
        const uint32_t kk = fkey(x[j]);
        if ((kk & mask) == prefix && IN_K(kk, i0 + j)) {
          amount = mass_of(c, x[j]);
          return (int)((kk >> shift) & 255u);
        }
        amount = 0;
        return -1;
      }, target, shift, prefix, above);
      mask |= 255u << shift;
    }
    const u64 need = target > above ? target - above : 1ull;
    u64 total;
    const int tie = cl.template find<VPT>(nv, i0, [&](int j) -> u64 {
      const uint32_t kk = fkey(x[j]);
      return (kk == prefix && IN_K(kk, i0 + j)) ? mass_of(c, x[j]) : 0ull;
    }, need, &total);
    cut_p.key = prefix;
    cut_p.tie_last = tie;
  }

  // ---------------- draw ----------------
  auto final_mass = [&](int j) -> u64 {
    const uint32_t kk = fkey(x[j]);
    return (IN_K(kk, i0 + j) && in_cut(cut_p, kk, i0 + j)) ? mass_of(c, x[j]) : 0ull;
  };
  u64 zsum = 0;
#pragma unroll
  for (int j = 0; j < VPT; ++j)
    if (j < nv) zsum += final_mass(j);
  zsum = cl.sum(zsum);
  float u = uniform[row];
  u = fminf(fmaxf(u, 0.f), 0.99999994f);
  u64 r = (u64)((double)zsum * (double)u);
  if (r >= zsum) r = zsum ? zsum - 1 : 0;
  u64 total;
  int drawn = zsum ? cl.template find<VPT>(nv, i0, final_mass, r + 1, &total) : -1;
  if (drawn == 0x7fffffff) drawn = -1;
#undef IN_K
  if (cl.rank == 0 && threadIdx.x == 0) {
    int tok = drawn;
    if (tok < 0) {
      // an empty set (a row without a finite value): fall back to the first maximum
      tok = 0;
      float bv = -INFINITY;
      for (int i = 0; i < V; ++i)
        if (c.x[i] > bv) {
          bv = c.x[i];
          tok = i;
        }
    }
    out[row] = tok;
  }
  cl.cluster.sync();            // no CTA leaves while another may still read its shared memory
}

template <int VPT>
int launch_sample_cluster(const float* logits, long long ld, int B, int V, const float* temperature, const int* top_k,
                          const float* top_p, const float* min_p, const float* uniform, int* out, cudaStream_t st) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(CS, B);
  cfg.blockDim = dim3(NT);
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = CS;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, sample_cluster_kernel<VPT>, logits, ld, V, temperature, top_k, top_p, min_p,
                                 uniform, out);
}

static int g_sample_cluster = 1;

}  // namespace

LK_API int lk_argmax(const float* logits, long long ld, int B, int V, int* out, void* stream) {
  if (B <= 0) return LKH_OK;
  argmax_kernel<<<B, NT, 0, (cudaStream_t)stream>>>(logits, ld, V, out);
  lkh::count_launch();
  return lkh::launch_status();
}

LK_API int lk_repeat_penalty(float* logits, long long ld, int B, int V, const int* recent, int L,
                             const float* penalty, void* stream) {
  if (B <= 0 || L <= 0) return LKH_OK;
  repeat_penalty_kernel<<<B, 128, 0, (cudaStream_t)stream>>>(logits, ld, V, recent, L, penalty);
  lkh::count_launch();
  return lkh::launch_status();
}

LK_API int lk_sample(const float* logits, long long ld, int B, int V, const float* temperature, const int* top_k,
                     const float* top_p, const float* min_p, const float* uniform, int* out, void* stream) {
  if (B <= 0) return LKH_OK;
  if (!temperature || !uniform) return LKH_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  // a cluster of eight CTAs per row while that fills the GPU no more than twice over (a CTA of 1024 threads
  // with its part of the row in registers occupies an SM); beyond, one CTA per row is as fast (128k logits,
  // top-p: 58 us against 270 us for one row, 64 against 296 for eight, 286 against 320 for sixty-four)
  if (g_sample_cluster && B * CS <= 2 * 148 && V <= CS * NT * 32) {
    const int rc = V <= CS * NT * 16
                       ? launch_sample_cluster<16>(logits, ld, B, V, temperature, top_k, top_p, min_p, uniform, out, st)
                       : launch_sample_cluster<32>(logits, ld, B, V, temperature, top_k, top_p, min_p, uniform, out, st);
    if (rc) return rc;
    lkh::count_launch();
    return lkh::launch_status();
  }
  sample_kernel<<<B, NT, 0, st>>>(logits, ld, V, temperature, top_k, top_p, min_p, uniform, out);
  lkh::count_launch();
  return lkh::launch_status();
}

// Measurement and test hook: 0 keeps every row on the one-CTA kernel.
LK_API void lk_sample_cluster(int on) { g_sample_cluster = on; }

LK_API int lk_token_rules(float* logits, long long ld, int B, int V, const int* ids, const float* vals,
                          const int* counts, const int* modes, int R, void* stream) {
  if (B <= 0) return LKH_OK;
  if (!ids || !vals || !counts || !modes || R <= 0 || R > RULES_MAX) return LKH_BAD_ARG;
  token_rules_kernel<<<B, 256, 0, (cudaStream_t)stream>>>(logits, ld, V, ids, vals, counts, modes, R);
  lkh::count_launch();
  return lkh::launch_status();
}

LK_API int lk_token_bitmask(float* logits, long long ld, int B, int V, const unsigned* bits, int words,
                            const int* has, void* stream) {
  if (B <= 0) return LKH_OK;
  if (!bits || words * 32 < V) return LKH_BAD_ARG;
  dim3 grid((words + 255) / 256, B);
  token_bitmask_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(logits, ld, V, bits, words, has);
  lkh::count_launch();
  return lkh::launch_status();
}
