// Fused per-head q/k RMSNorm + RoPE + paged KV write, one launch for prefill rows and decode
// rows alike.  One warp per (token, head) of the fused qkv row:
//   q heads: optional RMSNorm over the head, rotation, written to a dense bf16 q buffer
//   k heads: optional RMSNorm, rotation, written to the paged cache at slot[token]
//   v heads: written to the paged cache
// The cache is either bf16 or "q8": int8 codes [slot, n_kv, hd] with one f16 scale per 32
// values in a separate plane [slot, n_kv, hd/32] (the Q8_0 numerics, d = amax/127,
// q = round(v/d), laid out so code rows stay 16-byte aligned for vector and TMA loads).
// RoPE pairing: 0 = adjacent lanes (2i, 2i+1), 1 = half-split (i, i + rope_dim/2).
// The inverse-frequency table is computed on the host so Llama-3 frequency factors, linear
// scaling and YaRN all reduce to "a table and a magnitude factor".
//
// Counterparts in the reference: loken_prefill_qk_rope_kv_f16_kernel and
// loken_decode_qkv_warp_f16_kernel (cuda/fused_norm_f16.cu:576-902),
// quantize_q8_0_kv_paired_dev_slot (src/inference/cuda/quantized/kv_quantize.cu).
#include "common.cuh"
#include "host_common.h"
#include "loken_cuda.h"
#include "tc100.cuh"

using namespace lk;

namespace {

// 1 / rms of a token's whole query projection and of its whole key projection: out[t] = {q, k}.
__global__ void __launch_bounds__(256)
qk_rinv_kernel(const __nv_bfloat16* __restrict__ qkv, long long ld, int T, int q_cols, int k_cols, float eps,
               float* __restrict__ out) {
  pdl_launch();
  pdl_wait();
  __shared__ float red[32];
  const int t = blockIdx.x;
  const __nv_bfloat16* row = qkv + (long long)t * ld;
  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x; i < q_cols; i += 256) {
    const float v = bf2f(row[i]);
    sq += v * v;
  }
  for (int i = threadIdx.x; i < k_cols; i += 256) {
    const float v = bf2f(row[q_cols + i]);
    sk += v * v;
  }
  sq = block_sum(sq, red);
  sk = block_sum(sk, red);
  if (threadIdx.x == 0) {
    out[(long long)t * 2] = rsqrtf(sq / (float)q_cols + eps);
    out[(long long)t * 2 + 1] = rsqrtf(sk / (float)k_cols + eps);
  }
}

template <int HD>
__global__ void __launch_bounds__(128)
rope_kv_kernel(const __nv_bfloat16* __restrict__ qkv, long long ld, const int* __restrict__ pos,
               const int* __restrict__ slots, int T, int n_q, int n_kv, const float* __restrict__ q_norm_w,
               const float* __restrict__ k_norm_w, float eps, const float* __restrict__ inv_freq, int rope_dim,
               int pairing, float mscale, __nv_bfloat16* __restrict__ q_out, void* __restrict__ k_cache,
               void* __restrict__ v_cache, __half* __restrict__ k_scale, __half* __restrict__ v_scale,
               long long num_slots, int kv_q8, int* __restrict__ status, const float* __restrict__ wide_rinv) {
  pdl_launch();      // nothing is written before the wait: the kernel after this one may set up behind it
  pdl_wait();
  constexpr int EPL = HD / 32;  // values per lane
  __shared__ float sh[4][HD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = n_q + 2 * n_kv;
  const long long unit = (long long)blockIdx.x * 4 + warp;
  if (unit >= (long long)T * heads) return;
  const int t = (int)(unit / heads);
  const int h = (int)(unit % heads);
  const bool is_q = h < n_q;
  const bool is_k = !is_q && h < n_q + n_kv;
  const __nv_bfloat16* src = qkv + (long long)t * ld + (long long)h * HD;

  float v[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) v[e] = bf2f(src[lane * EPL + e]);

  const float* nw = is_q ? q_norm_w : (is_k ? k_norm_w : nullptr);
  if (nw) {
    float r;
    if (wide_rinv) {
      // the norm runs over all the query (key) heads of the token at once (OLMoE): its scale was computed by
      // qk_rinv_kernel, the weight has one entry per column of the projection
      r = wide_rinv[(long long)t * 2 + (is_q ? 0 : 1)];
      nw += (long long)(is_q ? h : h - n_q) * HD;
    } else {
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) ss += v[e] * v[e];
      ss = warp_sum(ss);
      r = rsqrtf(ss / (float)HD + eps);
    }
#pragma unroll
    for (int e = 0; e < EPL; ++e) v[e] = v[e] * r * nw[lane * EPL + e];
  }

  if (is_q || is_k) {
#pragma unroll
    for (int e = 0; e < EPL; ++e) sh[warp][lane * EPL + e] = v[e];
    __syncwarp();
    const float p = (float)pos[t];
    const int half = rope_dim >> 1;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const int d = lane * EPL + e;
      if (d < rope_dim) {
        int fi, partner;
        bool first;
        if (pairing == 0) {
          fi = d >> 1;
          partner = d ^ 1;
          first = (d & 1) == 0;
        } else {
          first = d < half;
          fi = first ? d : d - half;
          partner = first ? d + half : d - half;
        }
        float sn, cs;
        sincosf(p * inv_freq[fi], &sn, &cs);
        sn *= mscale;
        cs *= mscale;
        const float a = sh[warp][d], b = sh[warp][partner];
        v[e] = first ? (a * cs - b * sn) : (a * cs + b * sn);
      }
    }
  }

  if (is_q) {
    __nv_bfloat16* dst = q_out + ((long long)t * n_q + h) * HD + lane * EPL;
#pragma unroll
    for (int e = 0; e < EPL; ++e) dst[e] = f2bf(v[e]);
    return;
  }

  const long long slot = slots[t];
  if (slot < 0) return;  // padding row: nothing to store
  if (slot >= num_slots) {
    if (status && lane == 0) atomicCAS(status, 0, LK_ERR_BOUNDS | (1 << 8));
    return;
  }
  const int kvh = is_k ? h - n_q : h - n_q - n_kv;
  void* cache = is_k ? k_cache : v_cache;
  if (!kv_q8) {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(cache) + (slot * n_kv + kvh) * HD + lane * EPL;
#pragma unroll
    for (int e = 0; e < EPL; ++e) dst[e] = f2bf(v[e]);
    return;
  }
  // q8: what a bf16 cache would have held is what gets quantised
#pragma unroll
  for (int e = 0; e < EPL; ++e) v[e] = bf2f(f2bf(v[e]));
  float amax = 0.f;
#pragma unroll
  for (int e = 0; e < EPL; ++e) amax = fmaxf(amax, fabsf(v[e]));
  constexpr int LPB = 32 / EPL;  // lanes per 32-value block
#pragma unroll
  for (int o = LPB / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const __half dh = __float2half(amax * (1.f / 127.f));
  const float d = __half2float(dh);
  const float id = d > 0.f ? 1.f / d : 0.f;
  int8_t* codes = reinterpret_cast<int8_t*>(cache) + (slot * n_kv + kvh) * HD + lane * EPL;
  if (EPL == 4) {
    char4 c;
    c.x = (signed char)__float2int_rn(v[0] * id);
    c.y = (signed char)__float2int_rn(v[1] * id);
    c.z = (signed char)__float2int_rn(v[2] * id);
    c.w = (signed char)__float2int_rn(v[3] * id);
    *reinterpret_cast<char4*>(codes) = c;
  } else {
#pragma unroll
    for (int e = 0; e < EPL; ++e) codes[e] = (int8_t)__float2int_rn(v[e] * id);
  }
  if ((lane % LPB) == 0) {
    __half* sc = (is_k ? k_scale : v_scale) + (slot * n_kv + kvh) * (HD / 32) + lane / LPB;
    *sc = dh;
  }
}

// Gather a sequence's K and V out of the paged cache into dense bf16 buffers for the flash
// prefill kernel: K as [tok, n_kv, hd] and V transposed as [n_kv, hd, ld_tok] so both are
// K-major MMA operands.  One block per (token-tile of 32, kv head).
template <int HD>
__global__ void __launch_bounds__(256)
kv_gather_kernel(const void* __restrict__ k_cache, const void* __restrict__ v_cache,
                 const __half* __restrict__ k_scale, const __half* __restrict__ v_scale, int kv_q8, int n_kv,
                 const int* __restrict__ block_table, int max_blocks, int block_size,
                 const int* __restrict__ seq_of_tile, const int* __restrict__ tile_tok0,
                 const int* __restrict__ kv_len, const int* __restrict__ dst_off, __nv_bfloat16* __restrict__ k_out,
                 __nv_bfloat16* __restrict__ vt_out, long long ld_tok, long long num_slots) {
  __shared__ __nv_bfloat16 vt[HD][34];
  const int tile = blockIdx.x, kvh = blockIdx.y;
  const int seq = seq_of_tile[tile];
  const int tok0 = tile_tok0[tile];
  const int len = kv_len[seq];
  const long long off = dst_off[seq];
  const int nthr = 256;
  // each thread moves 4 values at a time: 32 tokens x HD values / 4
  for (int idx = threadIdx.x; idx < 32 * HD / 4; idx += nthr) {
    const int tl = idx / (HD / 4);
    const int d = (idx % (HD / 4)) * 4;
    const int tok = tok0 + tl;
    float kf[4] = {0, 0, 0, 0}, vf[4] = {0, 0, 0, 0};
    if (tok < len) {
      const long long blk = block_table[(long long)seq * max_blocks + tok / block_size];
      const long long slot = blk * block_size + tok % block_size;
      if (slot >= 0 && slot < num_slots) {
        const long long base = (slot * n_kv + kvh) * HD + d;
        if (kv_q8) {
          const char4 kc = *reinterpret_cast<const char4*>(reinterpret_cast<const int8_t*>(k_cache) + base);
          const char4 vc = *reinterpret_cast<const char4*>(reinterpret_cast<const int8_t*>(v_cache) + base);
          const long long sb = (slot * n_kv + kvh) * (HD / 32) + d / 32;
          const float kd = __half2float(k_scale[sb]), vd = __half2float(v_scale[sb]);
          kf[0] = kc.x * kd; kf[1] = kc.y * kd; kf[2] = kc.z * kd; kf[3] = kc.w * kd;
          vf[0] = vc.x * vd; vf[1] = vc.y * vd; vf[2] = vc.z * vd; vf[3] = vc.w * vd;
        } else {
          const __nv_bfloat16* kp = reinterpret_cast<const __nv_bfloat16*>(k_cache) + base;
          const __nv_bfloat16* vp = reinterpret_cast<const __nv_bfloat16*>(v_cache) + base;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            kf[e] = bf2f(kp[e]);
            vf[e] = bf2f(vp[e]);
          }
        }
      }
    }
    __nv_bfloat16* ko = k_out + ((off + tok) * n_kv + kvh) * HD + d;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      ko[e] = f2bf(kf[e]);
      vt[d + e][tl] = f2bf(vf[e]);
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < HD * 32; idx += nthr) {
    const int d = idx / 32, tl = idx % 32;
    vt_out[((long long)kvh * HD + d) * ld_tok + off + tok0 + tl] = vt[d][tl];
  }
}

// Context shift: the keys and values of n cache positions move from `src` slots to `dst` slots, and
// every key is turned by `delta[i]` positions on the way (negative when the window slides down after
// older tokens were discarded; zero for positions that only move).  A stored key already carries its
// rotation and the attention factor, so a pure rotation by delta * inv_freq re-phases it: dequantise
// the row, rotate its pairs, requantise with a fresh step.  Values are copied as stored.  One warp per
// (position, kv head).  src and dst must not overlap (the caller writes into fresh blocks).
template <int HD>
__global__ void __launch_bounds__(128)
kv_shift_kernel(void* __restrict__ k_cache, void* __restrict__ v_cache, __half* __restrict__ k_scale,
                __half* __restrict__ v_scale, const int* __restrict__ src, const int* __restrict__ dst,
                const int* __restrict__ delta, int n, int n_kv, const float* __restrict__ inv_freq, int rope_dim,
                int pairing, long long num_slots, int kv_q8, int* __restrict__ status) {
  constexpr int EPL = HD / 32;
  __shared__ float sh[4][HD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * 4 + warp;
  if (unit >= (long long)n * n_kv) return;
  const int t = (int)(unit / n_kv), h = (int)(unit % n_kv);
  const long long so = src[t], dn = dst[t];
  if (so < 0 || dn < 0 || so >= num_slots || dn >= num_slots) {
    if (status && lane == 0) atomicCAS(status, 0, LK_ERR_BOUNDS | (2 << 8));
    return;
  }
  const long long srow = (so * n_kv + h) * HD + lane * EPL, drow = (dn * n_kv + h) * HD + lane * EPL;
  constexpr int LPB = 32 / EPL;      // lanes per 32-value block
  float v[EPL];
  if (kv_q8) {
    const float d = __half2float(k_scale[(so * n_kv + h) * (HD / 32) + lane / LPB]);
    const int8_t* c = reinterpret_cast<const int8_t*>(k_cache) + srow;
#pragma unroll
    for (int e = 0; e < EPL; ++e) v[e] = (float)c[e] * d;
  } else {
    const __nv_bfloat16* c = reinterpret_cast<const __nv_bfloat16*>(k_cache) + srow;
#pragma unroll
    for (int e = 0; e < EPL; ++e) v[e] = bf2f(c[e]);
  }
  const float p = (float)delta[t];
  if (p != 0.f) {
#pragma unroll
    for (int e = 0; e < EPL; ++e) sh[warp][lane * EPL + e] = v[e];
    __syncwarp();
    const int half = rope_dim >> 1;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const int dd = lane * EPL + e;
      if (dd < rope_dim) {
        int fi, partner;
        bool first;
        if (pairing == 0) {
          fi = dd >> 1;
          partner = dd ^ 1;
          first = (dd & 1) == 0;
        } else {
          first = dd < half;
          fi = first ? dd : dd - half;
          partner = first ? dd + half : dd - half;
        }
        float sn, cs;
        sincosf(p * inv_freq[fi], &sn, &cs);
        const float a = sh[warp][dd], b = sh[warp][partner];
        v[e] = first ? (a * cs - b * sn) : (a * cs + b * sn);
      }
    }
  }
  if (kv_q8) {
#pragma unroll
    for (int e = 0; e < EPL; ++e) v[e] = bf2f(f2bf(v[e]));
    float amax = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) amax = fmaxf(amax, fabsf(v[e]));
#pragma unroll
    for (int o = LPB / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const __half dh = __float2half(amax * (1.f / 127.f));
    const float d = __half2float(dh);
    const float id = d > 0.f ? 1.f / d : 0.f;
    int8_t* c = reinterpret_cast<int8_t*>(k_cache) + drow;
#pragma unroll
    for (int e = 0; e < EPL; ++e) c[e] = (int8_t)__float2int_rn(v[e] * id);
    if ((lane % LPB) == 0) k_scale[(dn * n_kv + h) * (HD / 32) + lane / LPB] = dh;
    // values: codes and steps as they are
    const int8_t* vs = reinterpret_cast<const int8_t*>(v_cache) + srow;
    int8_t* vd = reinterpret_cast<int8_t*>(v_cache) + drow;
#pragma unroll
    for (int e = 0; e < EPL; ++e) vd[e] = vs[e];
    if ((lane % LPB) == 0)
      v_scale[(dn * n_kv + h) * (HD / 32) + lane / LPB] = v_scale[(so * n_kv + h) * (HD / 32) + lane / LPB];
  } else {
    __nv_bfloat16* c = reinterpret_cast<__nv_bfloat16*>(k_cache) + drow;
#pragma unroll
    for (int e = 0; e < EPL; ++e) c[e] = f2bf(v[e]);
    const __nv_bfloat16* vs = reinterpret_cast<const __nv_bfloat16*>(v_cache) + srow;
    __nv_bfloat16* vd = reinterpret_cast<__nv_bfloat16*>(v_cache) + drow;
#pragma unroll
    for (int e = 0; e < EPL; ++e) vd[e] = vs[e];
  }
}

}  // namespace

LK_API int lk_kv_shift(void* k_cache, void* v_cache, void* k_scale, void* v_scale, const int* src, const int* dst,
                       const int* delta, int n, int n_kv, int hd, const float* inv_freq, int rope_dim, int pairing,
                       long long num_slots, int kv_q8, int* status, void* stream) {
  if (n <= 0) return LKH_OK;
  if (!k_cache || !v_cache || !src || !dst || !delta || !inv_freq || (kv_q8 && (!k_scale || !v_scale))) return LKH_BAD_ARG;
  const long long units = (long long)n * n_kv;
  const unsigned grid = (unsigned)((units + 3) / 4);
  cudaStream_t st = (cudaStream_t)stream;
#define LK_SHIFT(HD)                                                                                          \
  kv_shift_kernel<HD><<<grid, 128, 0, st>>>(k_cache, v_cache, (__half*)k_scale, (__half*)v_scale, src, dst, delta, \
                                            n, n_kv, inv_freq, rope_dim, pairing, num_slots, kv_q8, status)
  if (hd == 128) LK_SHIFT(128);
  else if (hd == 64) LK_SHIFT(64);
  else if (hd == 256) LK_SHIFT(256);
  else return LKH_BAD_ARG;
#undef LK_SHIFT
  lkh::count_launch();
  return lkh::launch_status();
}

static int rope_kv_impl(const void* qkv, long long ld, const int* pos, const int* slots, int T, int n_q, int n_kv,
                        int hd, const float* q_norm_w, const float* k_norm_w, float eps, const float* inv_freq,
                        int rope_dim, int pairing, float mscale, void* q_out, void* k_cache, void* v_cache,
                        void* k_scale, void* v_scale, long long num_slots, int kv_q8, int* status, void* stream,
                        const float* wide_rinv) {
  if (T <= 0) return LKH_OK;
  const long long units = (long long)T * (n_q + 2 * n_kv);
  const unsigned grid = (unsigned)((units + 3) / 4);
  cudaStream_t st = (cudaStream_t)stream;
#define LK_ROPE(HD)                                                                                          \
  lkh::launch_pdl(rope_kv_kernel<HD>, dim3(grid), dim3(128), 0, st, (const __nv_bfloat16*)qkv, ld, pos, slots, T, \
                  n_q, n_kv, q_norm_w, k_norm_w, eps, inv_freq, rope_dim, pairing, mscale,                       \
                  (__nv_bfloat16*)q_out, k_cache, v_cache, (__half*)k_scale, (__half*)v_scale, num_slots,        \
                  kv_q8, status, wide_rinv)
  if (hd == 128) LK_ROPE(128);
  else if (hd == 64) LK_ROPE(64);
  else if (hd == 256) LK_ROPE(256);
  else return LKH_BAD_ARG;
#undef LK_ROPE
  lkh::count_launch();
  return lkh::launch_status();
}

LK_API int lk_rope_kv(const void* qkv, long long ld, const int* pos, const int* slots, int T, int n_q, int n_kv,
                      int hd, const float* q_norm_w, const float* k_norm_w, float eps, const float* inv_freq,
                      int rope_dim, int pairing, float mscale, void* q_out, void* k_cache, void* v_cache,
                      void* k_scale, void* v_scale, long long num_slots, int kv_q8, int* status, void* stream) {
  return rope_kv_impl(qkv, ld, pos, slots, T, n_q, n_kv, hd, q_norm_w, k_norm_w, eps, inv_freq, rope_dim, pairing, mscale,
                      q_out, k_cache, v_cache, k_scale, v_scale, num_slots, kv_q8, status, stream, nullptr);
}

// The same with the q / k norm taken over the token's whole projection (weights of n_q * hd and n_kv * hd entries):
// `rinv` [T, 2] f32 scratch receives the two scales first.
LK_API int lk_rope_kv_wide(const void* qkv, long long ld, const int* pos, const int* slots, int T, int n_q, int n_kv,
                           int hd, const float* q_norm_w, const float* k_norm_w, float eps, const float* inv_freq,
                           int rope_dim, int pairing, float mscale, void* q_out, void* k_cache, void* v_cache,
                           void* k_scale, void* v_scale, long long num_slots, int kv_q8, int* status, float* rinv,
                           void* stream) {
  if (T <= 0) return LKH_OK;
  if (!rinv || !q_norm_w || !k_norm_w) return LKH_BAD_ARG;
  lkh::launch_pdl(qk_rinv_kernel, dim3(T), dim3(256), 0, (cudaStream_t)stream, (const __nv_bfloat16*)qkv, ld, T, n_q * hd,
                  n_kv * hd, eps, rinv);
  lkh::count_launch();
  return rope_kv_impl(qkv, ld, pos, slots, T, n_q, n_kv, hd, q_norm_w, k_norm_w, eps, inv_freq, rope_dim, pairing, mscale,
                      q_out, k_cache, v_cache, k_scale, v_scale, num_slots, kv_q8, status, stream, rinv);
}

LK_API int lk_kv_gather(const void* k_cache, const void* v_cache, const void* k_scale, const void* v_scale,
                        int kv_q8, int n_kv, int hd, const int* block_table, int max_blocks, int block_size,
                        const int* seq_of_tile, const int* tile_tok0, int n_tiles, const int* kv_len,
                        const int* dst_off, void* k_out, void* vt_out, long long ld_tok, long long num_slots,
                        void* stream) {
  if (n_tiles <= 0) return LKH_OK;
  dim3 grid(n_tiles, n_kv);
  cudaStream_t st = (cudaStream_t)stream;
#define LK_GATHER(HD)                                                                                            \
  kv_gather_kernel<HD><<<grid, 256, 0, st>>>(k_cache, v_cache, (const __half*)k_scale, (const __half*)v_scale,    \
                                             kv_q8, n_kv, block_table, max_blocks, block_size, seq_of_tile,       \
                                             tile_tok0, kv_len, dst_off, (__nv_bfloat16*)k_out,                   \
                                             (__nv_bfloat16*)vt_out, ld_tok, num_slots)
  if (hd == 128) LK_GATHER(128);
  else if (hd == 64) LK_GATHER(64);
  else return LKH_BAD_ARG;
#undef LK_GATHER
  lkh::count_launch();
  return lkh::launch_status();
}
