// Tensor-core GEMM core for sm_100a: C[i, j] = sum_k A[i, k] * B[j, k]
//
//   A: [Ra, K] K-major, its rows ride the MMA M dimension (128 per CTA)
//   B: [Rb, K] K-major, its rows ride the MMA N dimension (BN per CTA, 16..256)
//   C is written through two element strides (out_sa for i, out_sb for j), so the same
//   kernel serves "tokens x weights" (prefill: A = activations) and the swapped decode form
//   (A = weight rows, B = the few token rows), where a batch of 16..256 tokens fills N exactly
//   and no tensor-core work is wasted on padding.
//
// Pipeline per CTA: warp 0 = TMA producer, warp 1 = MMA issuer (one elected lane, tcgen05.mma
// with both operands read from 128-byte-swizzled shared memory, accumulators in TMEM),
// warps 2.. = epilogue (tcgen05.ld -> registers -> global), and, for quantised weights, four
// more warps that expand A from its block format to bf16 straight into the swizzled tile
// (dequant.cuh) while B still arrives by TMA.
//
// KIND_BF16: bf16 operands, accumulated over all of K in one TMEM accumulator per unit.
// KIND_F8BLK: e4m3 operands with block scales as DeepSeek-style checkpoints define them
//   (weights: one f32 scale per 128x128 block; activations: one f32 scale per token per 128
//   values of K).  Those scales are not the hardware's 1x32 micro-scaling, so each 128-wide
//   K block is accumulated on its own in one of four TMEM accumulators and the epilogue warps
//   fold it into fp32 registers with (scale_a * scale_b) while the tensor core works on.
//
// Split-K: every split writes its fp32 partial tile to a workspace; the split that arrives last
// on the tile's counter sums the partials in split order (deterministic) and runs the epilogue;
// it leaves the counter at zero for the next launch.
//
// Grouped (mixture of experts): A holds E stacked weight matrices, B the token rows sorted by
// expert; a device-side tile list says which expert and which token rows each N tile covers.
#pragma once
#include "tc100.cuh"
#include "symm.cuh"
#include "dequant.cuh"
#include <cuda_bf16.h>

namespace lk {

enum { KIND_BF16 = 0, KIND_F8BLK = 1 };
enum { SCALE_NONE = 0, SCALE_WBLOCK = 1, SCALE_ACT_T = 2 };

struct GemmParams {
  int Ra, Rb, K;
  int a_box_rows;             // rows of the A operand's TMA box (128, or fewer when the whole matrix is shorter)
  long long out_sa, out_sb;   // element strides of the output for i (A row) and j (B row)
  void* out;                  // bf16 (or fp32 when out_fp32)
  int out_fp32;
  const float* bias;          // optional, indexed by i when bias_on_a else by j
  int bias_on_a;
  const __nv_bfloat16* residual;  // optional, same strides as out
  const float* a_scale;
  int a_mode;
  long long a_ld;
  const float* b_scale;
  int b_mode;
  long long b_ld;
  float* ws;                  // split-K workspace
  int* counters;              // one per split tile, zero between launches
  int* status;                // error word
  int tiles_a, tiles_b, splits;   // output tiles and the K split of the tiles past n_full
  int n_full;                     // leading tiles that run as whole-K units (a multiple of the grid)
  int nrem, rem_mt;               // gemm_mx: units past n_full and the weight tiles in each of them
  int a_tiled;                    // gemm_mx: the weights are stored tile-major (16 KB per 128 x 128 tile)
  long long* prof;                // gemm_mx: optional per-CTA wait counters
  // quantised A (AFMT != 0): code plane and scale plane, row pitches in bytes
  const uint8_t* aq;
  const uint8_t* aq_scale;
  long long aq_ld, aq_sld;
  // grouped mode: N tiles come from a device-side list
  const int* g_tile_expert;   // [n] expert of the tile
  const int* g_tile_row0;     // [n] first B row (sorted token row) of the tile
  const int* g_tile_rows;     // [n] live rows of the tile (<= BN)
  const int* g_ntiles;        // [1] number of tiles in the list
  int g_rows_per_expert;      // A rows (output features) of one expert; 0 = not grouped
  int fuse_ar;                // sum the output over the ranks of `sv` inside the epilogue
  SymmView sv;
};

// Bounds and offsets of the tile a thread is finishing.
struct TileCtx {
  int ra_end;        // first A row past the tile's matrix (p.Ra, or the end of the expert's rows)
  int rb_end;        // first B row past the tile's live rows
  int a_base;        // A row that maps to output feature 0 (expert * rows_per_expert)
};

__device__ __forceinline__ void epi_bar(int nthreads) {
  asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
}

template <int KIND>
struct GemmTraits {
  static constexpr int KB = (KIND == KIND_BF16) ? 64 : 128;  // K elements per stage = 128 bytes
  static constexpr int ESIZE = (KIND == KIND_BF16) ? 2 : 1;
  static constexpr int UMMA_K = (KIND == KIND_BF16) ? 16 : 32;
};

template <int KIND, int BN, int STAGES, int CSPLIT>
struct GemmSmem {
  static constexpr int A_BYTES = 128 * 128;
  static constexpr int B_BYTES = BN * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 512 + 1024;  // barriers + alignment slack
};

// Fused all-reduce, step 1: this rank's partial (bias included: only one rank carries it) goes,
// as bf16, into slot `rank` of every rank's receive area at the element offset it has in `out`.
template <int CH>
__device__ __forceinline__ void push_chunk(const GemmParams& p, const TileCtx& t, int half, int i, int j0,
                                           const float (&v)[CH], bool local_only = false) {
  if (i >= t.ra_end) return;
  const int world = local_only ? 1 : p.sv.world, me = p.sv.rank;   // r = 0 is this rank's own heap
  const int io = i - t.a_base;
  const float ba = (p.bias && p.bias_on_a) ? p.bias[i] : 0.f;
  if (p.out_sb == 1 && (j0 + CH <= t.rb_end) && ((p.out_sa & 7) == 0)) {
    const long long off = (long long)io * p.out_sa + j0;
#pragma unroll
    for (int c = 0; c < CH; c += 8) {
      uint4 ov;
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float a = v[c + 2 * e] + ba, b = v[c + 2 * e + 1] + ba;
        if (p.bias && !p.bias_on_a) {
          a += p.bias[j0 + c + 2 * e];
          b += p.bias[j0 + c + 2 * e + 1];
        }
        o2[e] = __floats2bfloat162_rn(a, b);
      }
      for (int r = 0; r < world; ++r) {
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(symm_recv(p.sv, (me + r) % p.sv.world, half, me));
        *reinterpret_cast<uint4*>(dst + off + c) = ov;
      }
    }
    return;
  }
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int j = j0 + c;
    if (j < t.rb_end) {
      float x = v[c] + ba;
      if (p.bias && !p.bias_on_a) x += p.bias[j];
      const long long off = (long long)io * p.out_sa + (long long)j * p.out_sb;
      const __nv_bfloat16 h = __float2bfloat16(x);
      for (int r = 0; r < world; ++r)
        reinterpret_cast<__nv_bfloat16*>(symm_recv(p.sv, (me + r) % p.sv.world, half, me))[off] = h;
    }
  }
}

// Fused all-reduce, step 2: sum of the world's partials for this thread's chunk, in rank order.
template <int CH>
__device__ __forceinline__ void reduce_chunk(const GemmParams& p, const TileCtx& t, int half, int i, int j0,
                                             float (&v)[CH]) {
#pragma unroll
  for (int c = 0; c < CH; ++c) v[c] = 0.f;
  if (i >= t.ra_end) return;
  const int world = p.sv.world, me = p.sv.rank;
  const int io = i - t.a_base;
  if (p.out_sb == 1 && (j0 + CH <= t.rb_end) && ((p.out_sa & 7) == 0)) {
    const long long off = (long long)io * p.out_sa + j0;
    for (int s = 0; s < world; ++s) {
      const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(symm_recv(p.sv, me, half, s)) + off;
#pragma unroll
      for (int c = 0; c < CH; c += 8) {
        const uint4 q = __ldcg(reinterpret_cast<const uint4*>(src + c));
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h[e]);
          v[c + 2 * e] += f.x;
          v[c + 2 * e + 1] += f.y;
        }
      }
    }
    return;
  }
  for (int s = 0; s < world; ++s) {
    const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(symm_recv(p.sv, me, half, s));
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int j = j0 + c;
      if (j < t.rb_end) v[c] += __bfloat162float(__ldcg(src + (long long)io * p.out_sa + (long long)j * p.out_sb));
    }
  }
}

// ---- fused all-reduce, whole-tile form -----------------------------------------------------
// The tile's region of the output is `rows` runs of `cols` contiguous bf16 (cols a multiple of
// 8, every run 16-byte aligned): element offset of run r is off0 + r * ld.  The epilogue threads
// walk it as 16-byte pieces, consecutive threads on consecutive pieces, so peer stores leave as
// whole 128..256-byte runs and every load of the sum is in flight at once.
struct FlatTile {
  long long off0, ld;
  int rows, cols;
  bool ok;
};
__device__ __forceinline__ FlatTile flat_tile(const GemmParams& p, const TileCtx& t, int a_row0, int b_row0, int bn) {
  FlatTile f;
  const int na = min(128, t.ra_end - a_row0), nb = min(bn, t.rb_end - b_row0);
  if (p.out_sb == 1) {            // tokens on A: runs along j
    f.off0 = (long long)a_row0 * p.out_sa + b_row0; f.ld = p.out_sa; f.rows = na; f.cols = nb;
  } else {                        // weights on A: runs along i
    f.off0 = (long long)b_row0 * p.out_sb + a_row0; f.ld = p.out_sb; f.rows = nb; f.cols = na;
  }
  f.ok = (p.out_sb == 1 || p.out_sa == 1) && p.g_rows_per_expert == 0 && ((f.ld & 7) == 0) &&
         ((f.off0 & 7) == 0) && ((f.cols & 7) == 0) && f.rows > 0 && f.cols > 0 &&
         ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0) && ((reinterpret_cast<uintptr_t>(p.residual) & 15) == 0);
  return f;
}
// Step 1b: this rank's tile, already in its own slot of its own heap, goes to the same slot of
// every peer.
template <int NT>
__device__ __forceinline__ void flat_push(const GemmParams& p, const FlatTile& f, int half, int tid) {
  const int world = p.sv.world, me = p.sv.rank;
  const int ppr = f.cols >> 3, pieces = f.rows * ppr;
  const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(symm_recv(p.sv, me, half, me));
  for (int q0 = tid; q0 < pieces; q0 += NT * 4) {
    uint4 v[4];
    long long off[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int q = q0 + u * NT;
      const int r = q / ppr;
      off[u] = f.off0 + (long long)r * f.ld + (q - r * ppr) * 8;
      if (q < pieces) v[u] = __ldcg(reinterpret_cast<const uint4*>(src + off[u]));
    }
    for (int r = 1; r < world; ++r) {
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(symm_recv(p.sv, (me + r) % world, half, me));
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (q0 + u * NT < pieces) *reinterpret_cast<uint4*>(dst + off[u]) = v[u];
    }
  }
}
// Step 2: the ranks' tiles are summed in rank order (fp32), the residual is added, bf16 out.
// W is the world size (a build per size keeps exactly W loads per piece in registers); PP pieces
// are in flight per thread.
template <int NT, int W>
__device__ __forceinline__ void flat_reduce_store_w(const GemmParams& p, const FlatTile& f, int half, int tid) {
  constexpr int PP = 8 / W;        // eight 16-byte loads in flight per thread, whatever the world size
  const int me = p.sv.rank;
  const int ppr = f.cols >> 3, pieces = f.rows * ppr;
  const __nv_bfloat16* slot0 = reinterpret_cast<const __nv_bfloat16*>(symm_recv(p.sv, me, half, 0));
  const long long sstride = p.sv.slot_bytes >> 1;
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out);
  for (int q0 = tid; q0 < pieces; q0 += NT * PP) {
    uint4 v[PP][W], res[PP];
    long long off[PP];
#pragma unroll
    for (int u = 0; u < PP; ++u) {
      const int q = q0 + u * NT;
      const int r = q / ppr;
      off[u] = f.off0 + (long long)r * f.ld + (q - r * ppr) * 8;
      res[u] = make_uint4(0u, 0u, 0u, 0u);
      if (q < pieces) {
#pragma unroll
        for (int s = 0; s < W; ++s) v[u][s] = __ldcg(reinterpret_cast<const uint4*>(slot0 + s * sstride + off[u]));
        if (p.residual) res[u] = __ldg(reinterpret_cast<const uint4*>(p.residual + off[u]));
      }
    }
#pragma unroll
    for (int u = 0; u < PP; ++u) {
      if (q0 + u * NT >= pieces) continue;
      float a[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) a[e] = 0.f;
#pragma unroll
      for (int s = 0; s < W; ++s) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[u][s]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 x = __bfloat1622float2(h[e]);
          a[2 * e] += x.x;
          a[2 * e + 1] += x.y;
        }
      }
      uint4 ov;
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
      const __nv_bfloat162* rh = reinterpret_cast<const __nv_bfloat162*>(&res[u]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 x = __bfloat1622float2(rh[e]);
        o2[e] = __floats2bfloat162_rn(a[2 * e] + x.x, a[2 * e + 1] + x.y);
      }
      *reinterpret_cast<uint4*>(out + off[u]) = ov;
    }
  }
}
template <int NT>
__device__ __forceinline__ void flat_reduce_store(const GemmParams& p, const FlatTile& f, int half, int tid) {
  switch (p.sv.world) {
    case 2: flat_reduce_store_w<NT, 2>(p, f, half, tid); return;
    case 4: flat_reduce_store_w<NT, 4>(p, f, half, tid); return;
    case 8: flat_reduce_store_w<NT, 8>(p, f, half, tid); return;
    default: break;
  }
  // any other world size: one piece at a time
  const int world = p.sv.world, me = p.sv.rank;
  const int ppr = f.cols >> 3, pieces = f.rows * ppr;
  const __nv_bfloat16* slot0 = reinterpret_cast<const __nv_bfloat16*>(symm_recv(p.sv, me, half, 0));
  const long long sstride = p.sv.slot_bytes >> 1;
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out);
  for (int q = tid; q < pieces; q += NT) {
    const int r = q / ppr;
    const long long off = f.off0 + (long long)r * f.ld + (q - r * ppr) * 8;
    float a[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) a[e] = 0.f;
    for (int s = 0; s <= world; ++s) {
      if (s == world && !p.residual) break;
      const uint4 x4 = s < world ? __ldcg(reinterpret_cast<const uint4*>(slot0 + s * sstride + off))
                                 : __ldg(reinterpret_cast<const uint4*>(p.residual + off));
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x4);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 x = __bfloat1622float2(h[e]);
        a[2 * e] += x.x;
        a[2 * e + 1] += x.y;
      }
    }
    uint4 ov;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int e = 0; e < 4; ++e) o2[e] = __floats2bfloat162_rn(a[2 * e], a[2 * e + 1]);
    *reinterpret_cast<uint4*>(out + off) = ov;
  }
}

// Final stage for one chunk of CH columns held by this thread (row i): bias, residual, store.
template <int CH>
__device__ __forceinline__ void store_chunk(const GemmParams& p, const TileCtx& t, int i, int j0,
                                            const float (&v)[CH], bool with_bias = true) {
  const float* pbias = with_bias ? p.bias : nullptr;
  if (i >= t.ra_end) return;
  const int io = i - t.a_base;
  if (p.out_sb == 1 && !p.out_fp32 && (j0 + CH <= t.rb_end) && ((p.out_sa & 7) == 0)) {
    // row-contiguous output: 16-byte vector stores
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (long long)io * p.out_sa + j0;
    const __nv_bfloat16* r = p.residual ? p.residual + (long long)io * p.out_sa + j0 : nullptr;
    const float ba = (pbias && p.bias_on_a) ? pbias[i] : 0.f;
#pragma unroll
    for (int c = 0; c < CH; c += 8) {
      float x[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        x[e] = v[c + e] + ba;
        if (pbias && !p.bias_on_a) x[e] += pbias[j0 + c + e];
      }
      if (r) {
        uint4 rv = *reinterpret_cast<const uint4*>(r + c);
        const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float2 f = __bfloat1622float2(r2[e]);
          x[2 * e] += f.x;
          x[2 * e + 1] += f.y;
        }
      }
      uint4 ov;
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
      for (int e = 0; e < 4; ++e) o2[e] = __floats2bfloat162_rn(x[2 * e], x[2 * e + 1]);
      *reinterpret_cast<uint4*>(o + c) = ov;
    }
    return;
  }
  const float ba = (pbias && p.bias_on_a) ? pbias[i] : 0.f;
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int j = j0 + c;
    if (j < t.rb_end) {
      float x = v[c] + ba;
      if (pbias && !p.bias_on_a) x += pbias[j];
      const long long off = (long long)io * p.out_sa + (long long)j * p.out_sb;
      if (p.residual) x += __bfloat162float(p.residual[off]);
      if (p.out_fp32)
        reinterpret_cast<float*>(p.out)[off] = x;
      else
        reinterpret_cast<__nv_bfloat16*>(p.out)[off] = __float2bfloat16(x);
    }
  }
}

// The same final stage for outputs whose contiguous dimension is the A row (weights on the MMA M side,
// out[token][feature]): a thread holds one feature and CH tokens, so storing from registers writes two
// bytes per lane into rows a whole pitch apart.  Here the four epilogue warps of a tile (128 features)
// lay the chunk out in shared memory as [token][128 features] bf16 and then write every token's 256
// bytes as sixteen 16-byte stores: whole 128-byte lines, two token rows per warp instruction.
// `stage` holds 2 x CH x 128 bf16 (double buffered by `parity`: one barrier per chunk); `et` is the
// thread's index among the 128 epilogue threads (= feature row of the tile).  All 128 threads call it.
template <int CH>
__device__ __forceinline__ bool store_t_ok(const GemmParams& p) {
  return p.out_sa == 1 && !p.out_fp32 && !p.residual && (p.out_sb & 7) == 0 &&
         (reinterpret_cast<uintptr_t>(p.out) & 15) == 0;
}
template <int CH>
__device__ __forceinline__ void store_chunk_t(const GemmParams& p, const TileCtx& t, int i0, int et, int j0,
                                              const float (&v)[CH], __nv_bfloat16* stage, int parity,
                                              long long* tq = nullptr) {
  const long long q0 = tq ? clock64() : 0;
  // the staging tile in 32-bit words: [token][64 words = 128 features]; odd token rows are rotated by 16
  // words so that the two rows a warp writes at once fall into different banks
  uint32_t* sw = reinterpret_cast<uint32_t*>(stage) + parity * (CH * 64);
  const uint32_t sw_s = smem_u32(sw);          // shared-window address: explicit st.shared / ld.shared below
  const int lane = et & 31;
  const int i = i0 + et;
  float ba = 0.f;
  if (p.bias && p.bias_on_a && i < t.ra_end) ba = p.bias[i];
  // neighbouring lanes hold neighbouring features: they swap one value per token pair, so the even lane
  // writes both features of the even token as one word and the odd lane those of the odd token
  const int odd = lane & 1;
  const int w = (et >> 1);                      // word of this lane pair within a token row
  // in three sweeps (all swaps, all packs, all stores), so that the latencies of a sweep overlap
  float mine[CH / 2], got[CH / 2];
#pragma unroll
  for (int e = 0; e < CH; e += 2) {
    float x0 = v[e] + ba, x1 = v[e + 1] + ba;
    if (p.bias && !p.bias_on_a) {
      if (j0 + e < t.rb_end) x0 += p.bias[j0 + e];
      if (j0 + e + 1 < t.rb_end) x1 += p.bias[j0 + e + 1];
    }
    mine[e / 2] = odd ? x1 : x0;
    got[e / 2] = odd ? x0 : x1;
  }
#pragma unroll
  for (int k = 0; k < CH / 2; ++k) got[k] = __shfl_xor_sync(0xffffffffu, got[k], 1);
  uint32_t pk[CH / 2];
#pragma unroll
  for (int k = 0; k < CH / 2; ++k) {
    const __nv_bfloat162 h = odd ? __floats2bfloat162_rn(got[k], mine[k]) : __floats2bfloat162_rn(mine[k], got[k]);
    pk[k] = *reinterpret_cast<const uint32_t*>(&h);
  }
  const uint32_t sw_row = sw_s + 4u * (odd * 64 + ((w + 16 * odd) & 63));
#pragma unroll
  for (int k = 0; k < CH / 2; ++k)
    asm volatile("st.shared.b32 [%0], %1;" ::"r"(sw_row + 4u * (2 * k * 64)), "r"(pk[k]) : "memory");
  const long long q1 = tq ? clock64() : 0;
  epi_bar(128);
  const long long q2 = tq ? clock64() : 0;
  const int f0 = (et & 15) * 8;                 // eight features = 16 bytes
  const int io = i0 - t.a_base + f0;
  if (i0 + f0 + 8 <= t.ra_end) {
    // all reads from the staging tile first, then the global stores
    constexpr int NR = CH / 8;
    uint4 q[NR];
#pragma unroll
    for (int k = 0; k < NR; ++k) {
      const int r = (et >> 4) + 8 * k;
      asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(q[k].x), "=r"(q[k].y), "=r"(q[k].z), "=r"(q[k].w)
                   : "r"(sw_s + 4u * (r * 64 + (((f0 >> 1) + 16 * (r & 1)) & 63))));
    }
#pragma unroll
    for (int k = 0; k < NR; ++k) {
      const int j = j0 + (et >> 4) + 8 * k;
      if (j < t.rb_end)
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.out) + (long long)j * p.out_sb + io) = q[k];
    }
    if (tq) {
      tq[1] += q1 - q0;
      tq[2] += q2 - q1;
      tq[3] += clock64() - q2;
    }
  } else if (i0 + f0 < t.ra_end) {
    // the last features of a matrix whose row count is not a multiple of eight
    for (int r = et >> 4; r < CH; r += 8) {
      const int j = j0 + r;
      if (j < t.rb_end) {
        const __nv_bfloat16* row = reinterpret_cast<const __nv_bfloat16*>(sw + r * 64 + (((f0 >> 1) + 16 * (r & 1)) & 63));
        for (int e = 0; e < 8 && i0 + f0 + e < t.ra_end; ++e)
          reinterpret_cast<__nv_bfloat16*>(p.out)[(long long)j * p.out_sb + io + e] = row[e];
      }
    }
  }
}

}  // namespace lk

#include "gemm_tc_kernel.cuh"
