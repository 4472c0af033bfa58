// Quantised GEMV for decode-size batches (1..8 token rows): out[m, n] = sum_k W[n, k] x[m, k] with W in a
// GGUF block format held as device planes (ops/quant.py: codes + scale records) and the activations
// quantised to int8 per 32 values on the fly, so the inner product is `dp4a` on the stored integer codes:
// nothing is expanded to bf16 and the weights are read exactly once.  This is the single-stream decode
// path of quantised models; from nine token rows up the tensor-core GEMM with dequantising warps
// (gemm_tc.cuh, dequant.cuh) takes over.
//
//   Q8_0   int8 codes, one f16 scale per 32 values
//   Q6_K   int8 codes (already centred), per 256 values: f16 d + sixteen int8 sub-scales (one per 16)
//   Q4_K   nibbles (value k in byte k / 2, low nibble for even k), per 256 values: f16 d, f16 dmin,
//          eight 6-bit sub-scales and eight 6-bit minima as bytes (one of each per 32 values)
//
// Layout of the work: a CTA first quantises the M activation rows into shared memory, once (int8 codes,
// one f32 scale and, for Q4_K, one f32 sum per 32 values: the minimum term needs sum(x)); from there on it
// has no barrier.  It then walks row groups (8 warps x RW rows) strided over the grid: a lane owns every
// 32nd group of 32 values of K, takes the M groups of activation codes from shared memory and reads 32
// weight codes per row (16 or 32 bytes) plus the group's scale fields; floats accumulate per (row, token),
// one butterfly per (row, token) ends a row group.  A first form that quantised 1024 values of K per
// step between two barriers spent most of its time in those steps (Q8_0, 57344 x 8192: 134 us at one
// token, 380 us at eight).
//
// The reference's quantised decode is the same idea with its own block layouts: int8 activations (q8_1) and
// dp4a over the codes (cuda/moe/moe_gguf.cu:405-1340, src/inference/cuda/quantized/); its accuracy bar for
// 8-bit activations is 2e-2 of the largest expected output.
#include "common.cuh"
#include "host_common.h"
#include "loken_cuda.h"
#include "tc100.cuh"

using namespace lk;

namespace {

constexpr int GV_WARPS = 8;
// GV_W4G: nibbles like GV_W4, per 128 values one f16 scale and one f16 minimum (= zero point x scale): AWQ's
// 4-bit weights with groups of 128 (w = (q - zero) * scale), repacked at load (ops/quant.py: from_awq)
enum { GV_W8 = 1, GV_W8G16 = 2, GV_W4 = 3, GV_W4G = 5 };
template <int FMT> __host__ __device__ constexpr bool gv_nibbles() { return FMT == GV_W4 || FMT == GV_W4G; }

__device__ __forceinline__ int dp4a_s8(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ int dp4a_u8s8(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
// hints: bring [p, p + bytes) (16-byte aligned, a multiple of 16 bytes) or the line of p into L2
__device__ __forceinline__ void l2_prefetch_bulk(const void* p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}
__device__ __forceinline__ void l2_prefetch_line(const void* p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ float h2f(const uint8_t* p) {
  return __half2float(*reinterpret_cast<const __half*>(p));
}

struct GvParams {
  const uint8_t* codes;       // [N, code bytes per row]
  const uint8_t* scales;      // [N, scale bytes per row]
  long long c_ld, s_ld;       // row pitches in bytes
  const __nv_bfloat16* x;     // [M, K]
  long long ldx;
  const float* bias;          // [N] or null
  __nv_bfloat16* out;         // [M, N] bf16, or f32 when out_fp32
  long long ldo;
  int M, N, K;
  int out_fp32;
  LkGemvPre pre;              // what the activations are computed from (plain rows, a norm, a gated unit)
  // expert slots (streaming form, one token row per slot): slot s (blockIdx.y) multiplies row s / slot_x_div of x
  // by the matrix of expert slot_expert[s] of a stack of [N, K] matrices and writes row s of out
  const int* slot_expert;
  int slots, slot_x_div, slot_e_lo, slot_e_cnt;
};

__device__ __forceinline__ void load8f(const __nv_bfloat16* src, float* v) {
  const uint4 u = *reinterpret_cast<const uint4*>(src);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 f = __bfloat1622float2(h[e]);
    v[2 * e] = f.x;
    v[2 * e + 1] = f.y;
  }
}
// Values 8 c .. 8 c + 7 of token row m of the residual stream as the norm sees it: x, plus the pending
// update rounded into bf16 the way the stream stores it.
__device__ __forceinline__ void residual8(const GvParams& p, long long x_off, int m, int c, float* v) {
  load8f(p.x + x_off + (long long)m * p.ldx + c * 8, v);
  if (p.pre.delta) {
    float d[8];
    load8f(reinterpret_cast<const __nv_bfloat16*>(p.pre.delta) + (long long)m * p.pre.ldd + c * 8, d);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = bf2f(f2bf(v[e] + d[e]));
  }
}

// Eight activations of token row m as the GEMV multiplies them: the rows of x themselves, or
// RMSNorm(x + delta) * gamma (rinv = 1 / rms of the row), or the gated unit of x = [gate | up]; each rounded
// to bf16 where the separate kernels store bf16.
__device__ __forceinline__ void activation8(const GvParams& p, long long x_off, int m, int c, float rinv, float* v) {
  if (p.pre.mode == 1) {
    residual8(p, x_off, m, c, v);
    const float4* g4 = reinterpret_cast<const float4*>(p.pre.gamma + c * 8);
    const float4 ga = g4[0], gb = g4[1];
    const float g[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = bf2f(f2bf(v[e] * rinv * g[e]));
  } else if (p.pre.mode == 2) {
    float u[8];
    load8f(p.x + x_off + (long long)m * p.ldx + c * 8, v);
    load8f(p.x + x_off + (long long)m * p.ldx + p.K + c * 8, u);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float o;
      if (p.pre.glu_mode == 0) {
        o = silu(v[e]) * u[e];
      } else {
        const float gg = fminf(v[e], p.pre.glu_limit);
        const float uu = fminf(fmaxf(u[e], -p.pre.glu_limit), p.pre.glu_limit);
        o = gg / (1.f + __expf(-p.pre.glu_alpha * gg)) * (1.f + uu);
      }
      v[e] = bf2f(f2bf(o));
    }
  } else {
    load8f(p.x + x_off + (long long)m * p.ldx + c * 8, v);
  }
}

// The activations of the M token rows, quantised once per CTA into shared memory by its 256 compute threads
// (threadIdx.x 0 .. 255; SYNC is the barrier those threads share): int8 codes as words (for Q4_K de-interleaved
// per 8 values, even values then odd ones, to line up with the nibble planes), one scale and one sum per group
// of 32.  A thread takes 8 values, four neighbouring lanes make a group: the phase sits between the kernel
// before this one and the first product, so it is spread over every thread rather than run as 128 serial
// groups.  With a norm in front, a first pass sums the squares of every row.  CTA 0 also applies a residual
// update that an earlier kernel of the step left pending (upd_x += upd_delta): every reader of the old rows
// finished with the kernel before this one.
template <int FMT, int MT, class SYNC>
__device__ __forceinline__ void stage_activations(const GvParams& p, long long x_off, uint32_t* xq, float* xd, float* xs,
                                                  int ngroups, SYNC sync) {
  __shared__ float s_red[GV_WARPS][8];
  __shared__ float s_rinv[8];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cpr = p.K >> 3;                        // chunks of 8 per row
  if (p.pre.upd_x && blockIdx.x == 0) {
    __nv_bfloat16* ux = reinterpret_cast<__nv_bfloat16*>(p.pre.upd_x);
    const __nv_bfloat16* ud = reinterpret_cast<const __nv_bfloat16*>(p.pre.upd_delta);
    const int per_row = p.pre.upd_cols >> 3;
    for (int i = tid; i < p.M * per_row; i += GV_WARPS * 32) {
      const int m = i / per_row, c = (i % per_row) * 8;
      uint4 a = *reinterpret_cast<const uint4*>(ux + (long long)m * p.pre.upd_ldx + c);
      const uint4 d = *reinterpret_cast<const uint4*>(ud + (long long)m * p.pre.upd_ldd + c);
      __nv_bfloat162* ah = reinterpret_cast<__nv_bfloat162*>(&a);
      const __nv_bfloat162* dh = reinterpret_cast<const __nv_bfloat162*>(&d);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 fa = __bfloat1622float2(ah[e]), fd = __bfloat1622float2(dh[e]);
        ah[e] = __floats2bfloat162_rn(fa.x + fd.x, fa.y + fd.y);
      }
      *reinterpret_cast<uint4*>(ux + (long long)m * p.pre.upd_ldx + c) = a;
    }
  }
  if (p.pre.mode == 1) {
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      float ss = 0.f;
      if (m < p.M)
#pragma unroll 4
        for (int c = tid; c < cpr; c += GV_WARPS * 32) {
          float v[8];
          residual8(p, x_off, m, c, v);
#pragma unroll
          for (int e = 0; e < 8; ++e) ss += v[e] * v[e];
        }
      ss = warp_sum(ss);
      if (lane == 0) s_red[warp][m] = ss;
    }
    sync();
    if (tid < MT) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < GV_WARPS; ++w) t += s_red[w][tid];
      s_rinv[tid] = rsqrtf(t / (float)p.K + p.pre.eps);
    }
    sync();
  }
  // chunks of a row are a multiple of four, so the four lanes of a group are in or out of range together;
  // every lane of a warp runs every trip (the shuffles below name the whole warp).  Four trips at a time: their
  // loads are all issued before the first value is used, so a batch costs one trip to L2 instead of four (the
  // phase took 3 us at K = 4096 and 7 us at K = 14336 with one load in flight per thread).
  constexpr int UB = 4;
  const int total = MT * cpr;
  for (int base = 0; base < total; base += UB * GV_WARPS * 32) {
    float v[UB][8];
#pragma unroll
    for (int u = 0; u < UB; ++u) {
      const int ch = base + u * GV_WARPS * 32 + tid;
      const int m = ch / cpr, c = ch % cpr;
      if (ch < total && m < p.M) {
        activation8(p, x_off, m, c, p.pre.mode == 1 ? s_rinv[m] : 1.f, v[u]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[u][e] = 0.f;
      }
    }
#pragma unroll
    for (int u = 0; u < UB; ++u) {
      const int ch = base + u * GV_WARPS * 32 + tid;
      const int m = ch / cpr, c = ch % cpr;
      float amax = 0.f, sum = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        amax = fmaxf(amax, fabsf(v[u][e]));
        sum += v[u][e];
      }
#pragma unroll
      for (int o = 1; o <= 2; o <<= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        sum += __shfl_xor_sync(0xffffffffu, sum, o);
      }
      const float d = amax * (1.f / 127.f);
      const float id = d > 0.f ? 1.f / d : 0.f;
      int q8[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) q8[e] = __float2int_rn(v[u][e] * id) & 0xFF;
      uint2 w;
      if (gv_nibbles<FMT>()) {
        w.x = q8[0] | (q8[2] << 8) | (q8[4] << 16) | (q8[6] << 24);
        w.y = q8[1] | (q8[3] << 8) | (q8[5] << 16) | (q8[7] << 24);
      } else {
        w.x = q8[0] | (q8[1] << 8) | (q8[2] << 16) | (q8[3] << 24);
        w.y = q8[4] | (q8[5] << 8) | (q8[6] << 16) | (q8[7] << 24);
      }
      if (ch < total) {
        *reinterpret_cast<uint2*>(xq + (size_t)m * (p.K >> 2) + c * 2) = w;
        if ((c & 3) == 0) {
          xd[m * ngroups + (c >> 2)] = d;
          xs[m * ngroups + (c >> 2)] = sum;
        }
      }
    }
  }
  sync();
}

// FMT: block format; MT: token rows (1, 2, 4 or 8); RW: output rows per warp and pass
template <int FMT, int MT, int RW>
__global__ void __launch_bounds__(GV_WARPS * 32)
gemv_q_kernel(const GvParams p) {
  // The weights do not depend on the kernel before this one, and this grid is resident while that kernel
  // still runs (programmatic launch).  So first ask for this CTA's rows to be brought into L2: the weights
  // of a decode step then stream through the stretches in which the small kernels between two GEMVs leave
  // the memory system idle, and the loads below find them on the chip.
  {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_rg = (p.N + GV_WARPS * RW - 1) / (GV_WARPS * RW);
    const uint32_t code_bytes = gv_nibbles<FMT>() ? p.K >> 1 : p.K;
    for (int rg = blockIdx.x; rg < n_rg; rg += gridDim.x) {
      const int row0 = (rg * GV_WARPS + warp) * RW;
      if (row0 >= p.N) continue;
      const int nrows = min(RW, p.N - row0);
      if (lane < nrows) l2_prefetch_bulk(p.codes + (long long)(row0 + lane) * p.c_ld, code_bytes);
      const uint8_t* sb = p.scales + (long long)row0 * p.s_ld;
      const long long span = (long long)nrows * p.s_ld;
      for (long long off = lane * 128ll; off < span; off += 32 * 128) l2_prefetch_line(sb + off);
    }
  }
  pdl_wait();
  pdl_launch();
  // the activations of the whole row, quantised once per CTA: codes as words (for Q4_K de-interleaved per 8
  // values, even values then odd ones, to line up with the nibble planes), scale and sum per 32-value group
  extern __shared__ __align__(128) uint8_t gv_smem[];
  const int ngroups = p.K >> 5;
  uint32_t* xq = reinterpret_cast<uint32_t*>(gv_smem);                         // [MT][K / 4]
  float* xd = reinterpret_cast<float*>(gv_smem + (size_t)MT * p.K);            // [MT][K / 32]
  float* xs = xd + MT * ngroups;                                               // [MT][K / 32]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  stage_activations<FMT, MT>(p, 0, xq, xd, xs, ngroups, [] { __syncthreads(); });

  // row groups of RW rows per warp, strided over the grid; no barrier from here on
  const int n_rg = (p.N + GV_WARPS * RW - 1) / (GV_WARPS * RW);
  for (int rg = blockIdx.x; rg < n_rg; rg += gridDim.x) {
    const int row0 = (rg * GV_WARPS + warp) * RW;
    if (row0 >= p.N) continue;
    float acc[RW][MT];
#pragma unroll
    for (int r = 0; r < RW; ++r)
#pragma unroll
      for (int m = 0; m < MT; ++m) acc[r][m] = 0.f;
    for (int gi = lane; gi < ngroups; gi += 32) {      // this lane's 32-value group of every chunk
      const int k = gi << 5;
      uint32_t xw[MT][8];
      float dx[MT], sx[MT];
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const uint4* src = reinterpret_cast<const uint4*>(xq + (size_t)m * (p.K >> 2) + gi * 8);
        const uint4 a = src[0], b = src[1];
        xw[m][0] = a.x; xw[m][1] = a.y; xw[m][2] = a.z; xw[m][3] = a.w;
        xw[m][4] = b.x; xw[m][5] = b.y; xw[m][6] = b.z; xw[m][7] = b.w;
        dx[m] = xd[m * ngroups + gi];
        sx[m] = xs[m * ngroups + gi];
      }
#pragma unroll
      for (int r = 0; r < RW; ++r) {
        const int n = min(row0 + r, p.N - 1);          // rows past the end repeat the last one; never stored
        if (FMT == GV_W8) {
          const uint4* c = reinterpret_cast<const uint4*>(p.codes + (long long)n * p.c_ld + k);
          const uint4 c0 = __ldcs(c), c1 = __ldcs(c + 1);
          const float dw = h2f(p.scales + (long long)n * p.s_ld + (k >> 5) * 2);
          const uint32_t cw[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            int s = 0;
#pragma unroll
            for (int q = 0; q < 8; ++q) s = dp4a_s8(cw[q], xw[m][q], s);
            acc[r][m] = fmaf(dw * dx[m], (float)s, acc[r][m]);
          }
        } else if (FMT == GV_W8G16) {
          const uint4* c = reinterpret_cast<const uint4*>(p.codes + (long long)n * p.c_ld + k);
          const uint4 c0 = __ldcs(c), c1 = __ldcs(c + 1);
          const uint8_t* rec = p.scales + (long long)n * p.s_ld + (k >> 8) * 18;
          const float d = h2f(rec);
          const int j = (k & 255) >> 4;                  // first of this group's two sub-scales
          const uint32_t two = *reinterpret_cast<const uint16_t*>(rec + 2 + j);      // j is even: 2-byte aligned
          const float s0 = d * (float)(int8_t)(two & 0xFF), s1 = d * (float)(int8_t)(two >> 8);
          const uint32_t cw[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            int a = 0, b = 0;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              a = dp4a_s8(cw[q], xw[m][q], a);
              b = dp4a_s8(cw[4 + q], xw[m][4 + q], b);
            }
            acc[r][m] = fmaf(dx[m], s0 * (float)a + s1 * (float)b, acc[r][m]);
          }
        } else {
          const uint4 c0 = __ldcs(reinterpret_cast<const uint4*>(p.codes + (long long)n * p.c_ld + (k >> 1)));
          float d, mn;
          if (FMT == GV_W4G) {
            const uint32_t dd = *reinterpret_cast<const uint32_t*>(p.scales + (long long)n * p.s_ld + (k >> 7) * 4);
            d = __half2float(__ushort_as_half((unsigned short)(dd & 0xFFFF)));
            mn = __half2float(__ushort_as_half((unsigned short)(dd >> 16)));
          } else {
            const uint8_t* rec = p.scales + (long long)n * p.s_ld + (k >> 8) * 20;
            const int j = (k & 255) >> 5;
            const uint32_t dd = *reinterpret_cast<const uint32_t*>(rec);        // d and dmin: records are 4-byte aligned
            d = __half2float(__ushort_as_half((unsigned short)(dd & 0xFFFF))) * (float)rec[4 + j];
            mn = __half2float(__ushort_as_half((unsigned short)(dd >> 16))) * (float)rec[12 + j];
          }
          const uint32_t cw[4] = {c0.x, c0.y, c0.z, c0.w};
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            int s = 0;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              s = dp4a_u8s8(cw[q] & 0x0F0F0F0Fu, xw[m][2 * q], s);              // even values
              s = dp4a_u8s8((cw[q] >> 4) & 0x0F0F0F0Fu, xw[m][2 * q + 1], s);   // odd values
            }
            acc[r][m] += d * dx[m] * (float)s - mn * sx[m];
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < RW; ++r) {
      const int n = row0 + r;
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const float v = warp_sum(acc[r][m]);
        if (lane == 0 && n < p.N && m < p.M) {
          const float o = v + (p.bias ? p.bias[n] : 0.f);
          if (p.out_fp32)
            reinterpret_cast<float*>(p.out)[(long long)m * p.ldo + n] = o;
          else
            p.out[(long long)m * p.ldo + n] = f2bf(o);
        }
      }
    }
  }
}

// ---- the streaming form ---------------------------------------------------------------------------------
// The form above keeps few bytes in flight: a lane's loads of one pass are all it has outstanding, and a
// GEMV of 10 to 60 MB took 10 to 22 us even with its weights already in L2.  Here a producer warp streams
// the CTA's rows through a ring of shared-memory stages with bulk asynchronous copies, so tens of KB per
// CTA are on their way at any time, and it does not wait for the kernel before this one (weights do not
// depend on it): by the time the activations exist the ring is full.
//
// A stage holds R whole rows (8, 4, 2 or 1: what fits 64 KB) and is filled by TWO copies, the rows' codes
// and the rows' scale records, both contiguous in their planes.  (A first form copied 2048 values of one
// row at a time, sixteen copies of 0.1 to 2 KB per stage: a stage then took 1.2 to 1.4 us whatever its
// size, the rate at which the copy engine takes requests.)  The eight consumer warps split a stage into
// R / RWP row groups times KS slices of K; a warp holds the activations of a group of 32 values in
// registers for its RWP rows.  Partial sums meet in shared memory, one barrier per stage.
// One group of 32 weights of one row (codes and scale records in shared memory: crow, srow) times the same
// group of every token row: acc[m] += w . x[m].  For Q4_K the high nibbles are multiplied where they stand
// (as multiples of 16) and the sum is shifted once: two logic operations per word instead of three.
template <int FMT, int MT>
__device__ __forceinline__ void row_dot(const uint8_t* crow, const uint8_t* srow, int g, const uint32_t (*xw)[8],
                                        const float* dx, const float* sx, float* acc) {
  if (FMT == GV_W8 || FMT == GV_W8G16) {
    const uint4* c = reinterpret_cast<const uint4*>(crow + g * 32);
    const uint4 c0 = c[0], c1 = c[1];
    const uint32_t cw[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    float s0, s1;
    if (FMT == GV_W8) {
      s0 = s1 = h2f(srow + g * 2);
    } else {
      const uint8_t* rec = srow + (g >> 3) * 18;
      const float d = h2f(rec);
      const uint32_t two = *reinterpret_cast<const uint16_t*>(rec + 2 + (g & 7) * 2);
      s0 = d * (float)(int8_t)(two & 0xFF);
      s1 = d * (float)(int8_t)(two >> 8);
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      int a = 0, b = 0;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        a = dp4a_s8(cw[q], xw[m][q], a);
        b = dp4a_s8(cw[4 + q], xw[m][4 + q], b);
      }
      acc[m] = fmaf(dx[m], s0 * (float)a + s1 * (float)b, acc[m]);
    }
  } else {
    const uint4 c0 = *reinterpret_cast<const uint4*>(crow + g * 16);
    float d, mn;
    if (FMT == GV_W4G) {
      const uint32_t dd = *reinterpret_cast<const uint32_t*>(srow + (g >> 2) * 4);
      d = __half2float(__ushort_as_half((unsigned short)(dd & 0xFFFF)));
      mn = __half2float(__ushort_as_half((unsigned short)(dd >> 16)));
    } else {
      const uint8_t* rec = srow + (g >> 3) * 20;
      const int j = g & 7;
      const uint32_t dd = *reinterpret_cast<const uint32_t*>(rec);
      d = __half2float(__ushort_as_half((unsigned short)(dd & 0xFFFF))) * (float)rec[4 + j];
      mn = __half2float(__ushort_as_half((unsigned short)(dd >> 16))) * (float)rec[12 + j];
    }
    const uint32_t cw[4] = {c0.x, c0.y, c0.z, c0.w};
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      int lo = 0, hi = 0;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        lo = dp4a_u8s8(cw[q] & 0x0F0F0F0Fu, xw[m][2 * q], lo);          // even values
        hi = dp4a_u8s8(cw[q] & 0xF0F0F0F0u, xw[m][2 * q + 1], hi);      // odd values, times 16
      }
      acc[m] += d * dx[m] * (float)(lo + (hi >> 4)) - mn * sx[m];
    }
  }
}

constexpr int GS_WARPS = 8;                 // consumer warps
constexpr int GS_THREADS = (GS_WARPS + 1) * 32;

template <int FMT>
__host__ __device__ constexpr int gs_code_bytes(int vals) { return gv_nibbles<FMT>() ? vals / 2 : vals; }
template <int FMT>
__host__ __device__ constexpr int gs_scale_bytes(int vals) {
  return FMT == GV_W8 ? vals / 16 : FMT == GV_W8G16 ? vals / 256 * 18 : FMT == GV_W4G ? vals / 128 * 4 : vals / 256 * 20;
}

__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(GS_WARPS * 32) : "memory"); }

// R: rows per stage; RWP: rows per warp; S: stages.  Row pitches equal the row sizes (contiguous planes).
// XR (one token row, at most two groups of K per lane): the lane's activation codes stay in registers for
// the whole kernel instead of being read from shared memory for every row.
template <int FMT, int MT, int R, int RWP, bool XR>
__global__ void __launch_bounds__(GS_THREADS)
gemv_q_stream_kernel(const GvParams p, int S, long long l2_budget, int* status) {
  static_assert(!XR || MT == 1, "activations in registers: one token row");
  // where this CTA's matrix, token row and output row start (an expert slot moves all of them)
  const uint8_t* codes = p.codes;
  const uint8_t* scales = p.scales;
  const float* bias = p.bias;
  long long x_off = 0, out_row0 = 0;
  if (p.slot_expert) {
    pdl_wait();                 // the expert of a slot is the routing kernel's output: nothing starts before it
    const int slot = blockIdx.y;
    const int e = p.slot_expert[slot] - p.slot_e_lo;
    if (e < 0 || e >= p.slot_e_cnt) return;           // another rank's expert
    codes += (long long)e * p.N * gs_code_bytes<FMT>(p.K);
    scales += (long long)e * p.N * gs_scale_bytes<FMT>(p.K);
    x_off = (long long)(slot / p.slot_x_div) * p.ldx;
    out_row0 = slot;
    if (bias) bias += (long long)e * p.N;
  }
  constexpr int NRG = R / RWP;             // row groups of a stage
  constexpr int KS = GS_WARPS / NRG;       // warps per row group, each takes every KS-th run of 32 groups
  static_assert(R % RWP == 0 && GS_WARPS % NRG == 0, "stage geometry");
  extern __shared__ __align__(128) uint8_t gv_smem[];
  const int ngroups = p.K >> 5;
  uint32_t* xq = reinterpret_cast<uint32_t*>(gv_smem);                         // [MT][K / 4]
  float* xd = reinterpret_cast<float*>(gv_smem + (size_t)MT * p.K);            // [MT][K / 32]
  float* xs = xd + MT * ngroups;                                               // [MT][K / 32]
  const int cb = gs_code_bytes<FMT>(p.K), sb = gs_scale_bytes<FMT>(p.K);       // bytes of a row in each plane
  const int pitch = (R * (cb + sb) + 127) & ~127;
  uint8_t* stages = gv_smem + (((size_t)MT * p.K + (size_t)MT * ngroups * 8 + 127) & ~(size_t)127);
  float* part = reinterpret_cast<float*>(stages + (size_t)S * pitch);          // [2][GS_WARPS][RWP * MT]
  uint64_t* full = reinterpret_cast<uint64_t*>(part + 2 * GS_WARPS * RWP * MT);
  uint64_t* empty = full + S;
  CtaAbort* ab = reinterpret_cast<CtaAbort*>(empty + S);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblk = (p.N + R - 1) / R;
  const int b0 = (int)((long long)blockIdx.x * nblk / gridDim.x);
  const int b1 = (int)((long long)(blockIdx.x + 1) * nblk / gridDim.x);
  const int nitems = b1 - b0;

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], GS_WARPS);
    }
    ab->flag = 0;
    fence_mbar_init();
  }
  __syncthreads();

  long long* prof = reinterpret_cast<long long*>(p.pre.prof);     // measurement hook: eight time stamps per CTA
  if (prof && threadIdx.x == 0) prof[blockIdx.x * 8 + 0] = (long long)globaltimer_ns();
  if (warp == GS_WARPS) {
    // ------------------------------ producer ------------------------------
    for (int it = 0; it < nitems; ++it) {
      const int s = it % S;
      if (it == S && l2_budget > 0) {
        // a measurement hook, off by default: the ring is full and its copies are on their way; what it cannot
        // hold yet is asked into L2 (up to this CTA's share of a budget that fits there).  The requests queue
        // in front of the activation loads of every CTA, whose staging phase then takes 5 us instead of 3:
        // a single-stream step of an 8B Q4_K_M model ran 4 to 5 % slower with the hints than without.
        const long long r0 = (long long)(b0 + S) * R, r1 = min((long long)p.N, (long long)b1 * R);
        const long long rows = min(r1 - r0, l2_budget / (cb + sb));
        const uint8_t* c0 = codes + r0 * cb;
        const uint8_t* s0 = scales + r0 * sb;
        for (long long off = lane * 4096ll; off < rows * cb; off += 32 * 4096)
          l2_prefetch_bulk(c0 + off, (uint32_t)min(4096ll, rows * cb - off));
        for (long long off = lane * 128ll; off < rows * sb; off += 32 * 128) l2_prefetch_line(s0 + off);
      }
      if (!mbar_wait(&empty[s], ((it / S) & 1) ^ 1, ab, status, 1)) break;
      const long long row0 = (long long)(b0 + it) * R;
      const int nvalid = (int)min((long long)R, p.N - row0);
      uint8_t* st = stages + (size_t)s * pitch;
      if (lane == 0) {
        if (prof && it == 0) prof[blockIdx.x * 8 + 5] = (long long)globaltimer_ns();
        if (prof && it == nitems - 1) prof[blockIdx.x * 8 + 6] = (long long)globaltimer_ns();
        mbar_expect_tx(&full[s], (uint32_t)(nvalid * (cb + sb)));
        bulk_g2s(st, codes + row0 * cb, (uint32_t)(nvalid * cb), &full[s]);
        bulk_g2s(st + R * cb, scales + row0 * sb, (uint32_t)(nvalid * sb), &full[s]);
      }
      __syncwarp();
    }
    return;
  }

  // ------------------------------ consumers ------------------------------
  pdl_wait();
  if (prof && threadIdx.x == 0) prof[blockIdx.x * 8 + 1] = (long long)globaltimer_ns();
  pdl_launch();
  stage_activations<FMT, MT>(p, x_off, xq, xd, xs, ngroups, [] { consumer_sync(); });
  if (prof && threadIdx.x == 0) prof[blockIdx.x * 8 + 2] = (long long)globaltimer_ns();

  const int rgp = warp / KS, ks = warp % KS;
  // XR: this lane's (at most two) groups of K, fixed for every row it will see
  uint32_t xr[2][8];
  float dxr[2], sxr[2];
  if (XR) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int g = ks * 32 + lane + i * KS * 32;
      if (g < ngroups) {
        const uint4* src = reinterpret_cast<const uint4*>(xq + g * 8);
        const uint4 a = src[0], b = src[1];
        xr[i][0] = a.x; xr[i][1] = a.y; xr[i][2] = a.z; xr[i][3] = a.w;
        xr[i][4] = b.x; xr[i][5] = b.y; xr[i][6] = b.z; xr[i][7] = b.w;
        dxr[i] = xd[g];
        sxr[i] = xs[g];
      } else {
#pragma unroll
        for (int q = 0; q < 8; ++q) xr[i][q] = 0;
        dxr[i] = sxr[i] = 0.f;
      }
    }
  }
  bool dead = false;                       // a wait gave up: no more waits, but every barrier below is still met
  for (int it = 0; it < nitems; ++it) {
    const int s = it % S;
    if (!dead && !mbar_wait(&full[s], (it / S) & 1, ab, status, 2)) dead = true;
    if (prof && threadIdx.x == 0 && it == 0) prof[blockIdx.x * 8 + 3] = (long long)globaltimer_ns();
    const long long row0 = (long long)(b0 + it) * R;
    const uint8_t* st = stages + (size_t)s * pitch;
    const uint8_t* cbase = st + (size_t)(rgp * RWP) * cb;
    const uint8_t* sbase = st + (size_t)R * cb + (size_t)(rgp * RWP) * sb;
    // rows of this warp that exist (the copy did not write rows past the matrix)
    const int live = dead ? 0 : (int)min((long long)RWP, p.N - (row0 + rgp * RWP));
    float acc[RWP][MT];
#pragma unroll
    for (int r = 0; r < RWP; ++r)
#pragma unroll
      for (int m = 0; m < MT; ++m) acc[r][m] = 0.f;
    if (XR) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int g = ks * 32 + lane + i * KS * 32;
        if (g < ngroups) {
#pragma unroll
          for (int r = 0; r < RWP; ++r)
            if (r < live)
              row_dot<FMT, 1>(cbase + (size_t)r * cb, sbase + (size_t)r * sb, g, &xr[i], &dxr[i], &sxr[i], acc[r]);
        }
      }
    } else {
#pragma unroll(MT <= 2 ? 2 : 1)
      for (int g = ks * 32 + lane; g < (live > 0 ? ngroups : 0); g += KS * 32) {
        uint32_t xw[MT][8];
        float dx[MT], sx[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          const uint4* src = reinterpret_cast<const uint4*>(xq + (size_t)m * (p.K >> 2) + g * 8);
          const uint4 a = src[0], b = src[1];
          xw[m][0] = a.x; xw[m][1] = a.y; xw[m][2] = a.z; xw[m][3] = a.w;
          xw[m][4] = b.x; xw[m][5] = b.y; xw[m][6] = b.z; xw[m][7] = b.w;
          dx[m] = xd[m * ngroups + g];
          sx[m] = xs[m * ngroups + g];
        }
#pragma unroll
        for (int r = 0; r < RWP; ++r)
          if (r < live) row_dot<FMT, MT>(cbase + (size_t)r * cb, sbase + (size_t)r * sb, g, xw, dx, sx, acc[r]);
      }
    }
    __syncwarp();
    if (lane == 0 && !dead) mbar_arrive(&empty[s]);      // the stage has been read
    float* mine = part + ((size_t)(it & 1) * GS_WARPS + warp) * (RWP * MT);
#pragma unroll
    for (int r = 0; r < RWP; ++r)
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const float v = warp_sum(acc[r][m]);
        if (lane == 0) mine[r * MT + m] = v;
      }
    consumer_sync();
    // the buffer of this parity is written again two stages on, after the barrier of the next stage, which
    // no thread passes before every reader below is done
    if (threadIdx.x < R * MT) {
      const int row = threadIdx.x / MT, m = threadIdx.x % MT;
      const int g2 = row / RWP, rr = row % RWP;
      const float* src = part + ((size_t)(it & 1) * GS_WARPS + g2 * KS) * (RWP * MT) + rr * MT + m;
      float v = 0.f;
#pragma unroll
      for (int k = 0; k < KS; ++k) v += src[k * (RWP * MT)];
      const long long n = row0 + row;
      if (n < p.N && m < p.M) {
        const float o = v + (bias ? bias[n] : 0.f);
        if (p.out_fp32)
          reinterpret_cast<float*>(p.out)[(out_row0 + m) * p.ldo + n] = o;
        else
          p.out[(out_row0 + m) * p.ldo + n] = f2bf(o);
      }
    }
  }
  if (prof && threadIdx.x == 0) prof[blockIdx.x * 8 + 4] = (long long)globaltimer_ns();
  if (ab->flag && threadIdx.x == 0) {
    // a wait gave up: give the copies still on their way a bounded time (0.2 ms) to land before the CTA leaves
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
}

static int g_gemv_stream = 1;

template <int FMT, int MT, int R, bool XR>
int launch_gs_x(const GvParams& p, cudaStream_t st, int* status, bool dry) {
  // rows per warp: as many as leave every lane of the warps that share a row group a group of K (R = 8:
  // four rows, four warps per group; shorter stages come with long rows)
  constexpr int RWP = R == 8 ? 4 : R >= 2 ? 2 : 1;
  const size_t row = (size_t)gs_code_bytes<FMT>(p.K) + gs_scale_bytes<FMT>(p.K);
  const size_t xbytes = ((size_t)MT * p.K + (size_t)MT * (p.K >> 5) * 8 + 127) & ~(size_t)127;
  const size_t pitch = ((size_t)R * row + 127) & ~(size_t)127;
  const size_t fixed = xbytes + 2 * GS_WARPS * RWP * MT * sizeof(float) + 12 * 16 + 16;
  // two CTAs per SM when the ring is at least three stages deep within half of the shared memory, else one
  size_t budget = 100 * 1024;
  if (fixed + 3 * pitch > budget) budget = 200 * 1024;
  if (fixed + 2 * pitch > budget) return -1;
  int S = (int)((budget - fixed) / pitch);
  if (S > 12) S = 12;
  const size_t smem = fixed + (size_t)S * pitch;
  if (dry) return 0;
  auto kern = gemv_q_stream_kernel<FMT, MT, R, RWP, XR>;
  static bool granted = false;
  if (!granted) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 201 * 1024);
    if (e != cudaSuccess) return (int)e;
    granted = true;
  }
  const int nblk = (p.N + R - 1) / R;
  const int per_sm = budget > 100 * 1024 ? 1 : 2;
  int grid = nblk < 148 * per_sm ? nblk : 148 * per_sm;
  int grid_y = 1;
  if (p.slot_expert) {
    // the slots share the SMs: each gets its part of the CTAs, at least one
    grid_y = p.slots;
    const int share = (148 * per_sm) / p.slots;
    grid = share < 1 ? 1 : (nblk < share ? nblk : share);
  }
  const long long l2_budget = ((g_gemv_stream & 2) && !p.slot_expert) ? (64ll << 20) / grid : 0;
  lkh::launch_pdl(kern, dim3(grid, grid_y), dim3(GS_THREADS), smem, st, p, S, l2_budget, status);
  return 0;
}

template <int FMT, int MT, int R>
int launch_gs_r(const GvParams& p, cudaStream_t st, int* status, bool dry) {
  constexpr int RWP = R == 8 ? 4 : R >= 2 ? 2 : 1;
  constexpr int KS = GS_WARPS / (R / RWP);
  if (MT == 1 && (p.K >> 5) <= 2 * KS * 32) return launch_gs_x<FMT, 1, R, true>(p, st, status, dry);
  return launch_gs_x<FMT, MT, R, false>(p, st, status, dry);
}

// Takes the shape when both planes are contiguous and every copy starts and ends on 16 bytes.
template <int FMT, int MT>
int launch_gs(const GvParams& p, cudaStream_t st, int* status, bool* taken, bool dry = false) {
  *taken = false;
  if (!g_gemv_stream || (!status && !dry)) return 0;
  // eight consumer warps are too few once every group of weights meets four or more token rows: there the
  // register form (24 warps per SM) is as fast or faster, except for the 8-bit planes at up to four rows
  // (Q6_K 4096 x 14336 at four rows: 25 us here, 33 us there; Q4_K 28672 x 4096: 46 us here, 32 us there)
  if (MT > 4 || (MT == 4 && gv_nibbles<FMT>())) return 0;
  const long long cb = gs_code_bytes<FMT>(p.K), sb = gs_scale_bytes<FMT>(p.K);
  if (p.c_ld != cb || p.s_ld != sb || (reinterpret_cast<uintptr_t>(p.scales) & 15)) return 0;
  // rows per stage: eight or four when a ring of three such stages fits half of an SM's shared memory (two
  // CTAs, sixteen consumer warps per SM: Q4_K 57344 x 8192 took 71 us with one CTA per SM and stages of eight
  // rows); else as many as fit 64 KB, one CTA per SM
  const size_t xb = (size_t)MT * p.K + (size_t)MT * (p.K >> 5) * 8 + 2048;
  int R = 8;
  while (R > 4 && xb + 3 * (size_t)R * (cb + sb) > 100 * 1024) R >>= 1;
  if (xb + 3 * (size_t)R * (cb + sb) > 100 * 1024) {
    R = 8;
    while (R > 1 && (size_t)R * (cb + sb) > 64 * 1024) R >>= 1;
    if ((size_t)R * (cb + sb) > 64 * 1024) return 0;
  }
  const long long tail = p.N % R;
  if (((R * cb) & 15) || ((R * sb) & 15) || ((tail * cb) & 15) || ((tail * sb) & 15)) return 0;
  if (p.slot_expert && ((p.N * sb) & 15)) return 0;      // every expert's scale plane starts on 16 bytes
  int rc;
  switch (R) {
    case 8: rc = launch_gs_r<FMT, MT, 8>(p, st, status, dry); break;
    case 4: rc = launch_gs_r<FMT, MT, 4>(p, st, status, dry); break;
    case 2: rc = launch_gs_r<FMT, MT, 2>(p, st, status, dry); break;
    default: rc = launch_gs_r<FMT, MT, 1>(p, st, status, dry); break;
  }
  if (rc < 0) return 0;            // does not fit: the register form takes it
  if (rc == 0) *taken = true;
  return rc;
}

template <int FMT, int MT>
int launch_gv(const GvParams& p, cudaStream_t st) {
  constexpr int RW = MT <= 2 ? 4 : 2;
  const size_t smem = (size_t)MT * p.K + (size_t)MT * (p.K >> 5) * 8;
  if (smem > 200 * 1024) return LKH_TOO_LARGE;
  auto kern = gemv_q_kernel<FMT, MT, RW>;
  static size_t granted = 48 * 1024;
  if (smem > granted) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return (int)e;
    granted = 200 * 1024;
  }
  // every CTA quantises the activations once, then walks row groups: a few CTAs per SM, not one per group
  const int n_rg = (p.N + GV_WARPS * RW - 1) / (GV_WARPS * RW);
  const int per_sm = smem > 100 * 1024 ? 1 : smem > 48 * 1024 ? 2 : 3;
  // every CTA walks the same number of row groups (a capped grid with a remainder leaves most SMs idle for
  // the last pass: 896 groups over 444 CTAs are two passes plus a third for eight of them)
  const int passes = (n_rg + 148 * per_sm - 1) / (148 * per_sm);
  const int grid = (n_rg + passes - 1) / passes;
  lkh::launch_pdl(kern, dim3(grid), dim3(GV_WARPS * 32), smem, st, p);
  return 0;
}

template <int FMT, int MT>
int launch_either(const GvParams& p, cudaStream_t st, int* status) {
  bool taken = false;
  const int rc = launch_gs<FMT, MT>(p, st, status, &taken);
  if (rc || taken) return rc;
  return launch_gv<FMT, MT>(p, st);
}

template <int FMT>
int dispatch_gv(const GvParams& p, int M, cudaStream_t st, int* status) {
  if (M == 1) return launch_either<FMT, 1>(p, st, status);
  if (M == 2) return launch_either<FMT, 2>(p, st, status);
  if (M <= 4) return launch_either<FMT, 4>(p, st, status);
  return launch_either<FMT, 8>(p, st, status);
}

// Embedding gather from a quantised table: row tok[t] of the planes is decoded to bf16.  One CTA per token,
// a thread per 32-value group and pass.
template <int FMT>
__global__ void __launch_bounds__(128)
embed_q_kernel(const int* __restrict__ tok, const uint8_t* __restrict__ codes, long long c_ld,
               const uint8_t* __restrict__ scales, long long s_ld, __nv_bfloat16* __restrict__ out, int H, int vocab,
               float scale) {
  const int t = blockIdx.x;
  int id = tok[t];
  if (id < 0 || id >= vocab) id = 0;
  const uint8_t* c = codes + (long long)id * c_ld;
  const uint8_t* s = scales + (long long)id * s_ld;
  __nv_bfloat16* dst = out + (long long)t * H;
  for (int g = threadIdx.x; g < (H >> 5); g += blockDim.x) {
    const int k = g << 5;
    float v[32];
    if (FMT == GV_W8) {
      const float d = h2f(s + g * 2) * scale;
      const int8_t* q = reinterpret_cast<const int8_t*>(c + k);
#pragma unroll
      for (int e = 0; e < 32; ++e) v[e] = d * (float)q[e];
    } else if (FMT == GV_W8G16) {
      const uint8_t* rec = s + (k >> 8) * 18;
      const float d = h2f(rec) * scale;
      const int j = (k & 255) >> 4;
      const float s0 = d * (float)(int8_t)rec[2 + j], s1 = d * (float)(int8_t)rec[3 + j];
      const int8_t* q = reinterpret_cast<const int8_t*>(c + k);
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        v[e] = s0 * (float)q[e];
        v[16 + e] = s1 * (float)q[16 + e];
      }
    } else {
      const uint8_t* rec = s + (k >> 8) * 20;
      const int j = (k & 255) >> 5;
      const float d = h2f(rec) * (float)rec[4 + j] * scale, mn = h2f(rec + 2) * (float)rec[12 + j] * scale;
      const uint8_t* q = c + (k >> 1);
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        v[2 * e] = d * (float)(q[e] & 0xF) - mn;
        v[2 * e + 1] = d * (float)(q[e] >> 4) - mn;
      }
    }
#pragma unroll
    for (int e = 0; e < 32; ++e) dst[k + e] = f2bf(v[e]);
  }
}

// The whole matrix decoded to bf16 [rows, K] (row pitch ldo elements): what a prompt-sized GEMM multiplies by.
// A thread decodes one group of 32 values (16 or 32 code bytes in, 64 bytes out); groups are walked in
// storage order, so a warp reads and writes contiguous runs.
template <int FMT>
__global__ void __launch_bounds__(256)
dequant_q_kernel(const uint8_t* __restrict__ codes, long long c_ld, const uint8_t* __restrict__ scales, long long s_ld,
                 __nv_bfloat16* __restrict__ out, long long ldo, int rows, int K) {
  pdl_wait();
  pdl_launch();
  const int ngroups = K >> 5;
  const long long total = (long long)rows * ngroups;
  for (long long g = blockIdx.x * 256ll + threadIdx.x; g < total; g += (long long)gridDim.x * 256) {
    const int n = (int)(g / ngroups), gi = (int)(g % ngroups);
    const int k = gi << 5;
    const uint8_t* c = codes + (long long)n * c_ld;
    const uint8_t* s = scales + (long long)n * s_ld;
    float v[32];
    if (FMT == GV_W8 || FMT == GV_W8G16) {
      const uint4* cp = reinterpret_cast<const uint4*>(c + k);
      const uint4 c0 = __ldg(cp), c1 = __ldg(cp + 1);
      const uint32_t cw[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
      float s0, s1;
      if (FMT == GV_W8) {
        s0 = s1 = h2f(s + gi * 2);
      } else {
        const uint8_t* rec = s + (k >> 8) * 18;
        const float d = h2f(rec);
        const int j = (k & 255) >> 4;
        s0 = d * (float)(int8_t)rec[2 + j];
        s1 = d * (float)(int8_t)rec[3 + j];
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float sc = q < 4 ? s0 : s1;
#pragma unroll
        for (int e = 0; e < 4; ++e) v[q * 4 + e] = sc * (float)(int8_t)((cw[q] >> (8 * e)) & 0xFF);
      }
    } else {
      const uint4 c0 = __ldg(reinterpret_cast<const uint4*>(c + (k >> 1)));
      float d, mn;
      if (FMT == GV_W4G) {
        d = h2f(s + (k >> 7) * 4);
        mn = h2f(s + (k >> 7) * 4 + 2);
      } else {
        const uint8_t* rec = s + (k >> 8) * 20;
        const int j = (k & 255) >> 5;
        d = h2f(rec) * (float)rec[4 + j];
        mn = h2f(rec + 2) * (float)rec[12 + j];
      }
      const uint32_t cw[4] = {c0.x, c0.y, c0.z, c0.w};
#pragma unroll
      for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const uint32_t b = (cw[q] >> (8 * e)) & 0xFF;
          v[q * 8 + 2 * e] = d * (float)(b & 0xF) - mn;
          v[q * 8 + 2 * e + 1] = d * (float)(b >> 4) - mn;
        }
    }
    uint4* dst = reinterpret_cast<uint4*>(out + (long long)n * ldo + k);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(v[q * 8 + 2 * e], v[q * 8 + 2 * e + 1]);
        w[e] = *reinterpret_cast<const uint32_t*>(&h);
      }
      dst[q] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

}  // namespace

// Planes of format fmt (1 Q8_0, 2 Q6_K, 3 Q4_K) decoded to bf16 out [rows, K], row pitch ldo elements (a
// multiple of 8, base 16-byte aligned).
LK_API int lk_dequant_q(int fmt, const void* codes, long long c_ld, const void* scales, long long s_ld, void* out,
                        long long ldo, int rows, int K, void* stream) {
  if (rows <= 0 || K <= 0) return LKH_OK;
  if (!codes || !scales || !out || (K & 31) || (ldo & 7) || ((fmt == GV_W8G16 || fmt == GV_W4) && (K & 255)) ||
      (fmt == GV_W4G && (K & 127)))
    return LKH_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(codes) & 15) || (c_ld & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return LKH_BAD_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const uint8_t* c = reinterpret_cast<const uint8_t*>(codes);
  const uint8_t* s = reinterpret_cast<const uint8_t*>(scales);
  __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out);
  const long long total = (long long)rows * (K >> 5);
  const long long want = (total + 255) / 256;
  const dim3 grid((unsigned)(want < 148 * 16 ? want : 148 * 16));
  switch (fmt) {
    case GV_W8: lkh::launch_pdl(dequant_q_kernel<GV_W8>, grid, dim3(256), 0, st, c, c_ld, s, s_ld, o, ldo, rows, K); break;
    case GV_W8G16: lkh::launch_pdl(dequant_q_kernel<GV_W8G16>, grid, dim3(256), 0, st, c, c_ld, s, s_ld, o, ldo, rows, K); break;
    case GV_W4: lkh::launch_pdl(dequant_q_kernel<GV_W4>, grid, dim3(256), 0, st, c, c_ld, s, s_ld, o, ldo, rows, K); break;
    case GV_W4G: lkh::launch_pdl(dequant_q_kernel<GV_W4G>, grid, dim3(256), 0, st, c, c_ld, s, s_ld, o, ldo, rows, K); break;
    default: return LKH_BAD_ARG;
  }
  lkh::count_launch();
  return lkh::launch_status();
}

// Rows tok[0 .. T) of a quantised embedding table (planes of format fmt: 1 Q8_0, 2 Q6_K, 3 Q4_K) decoded to
// bf16 out [T, H], times `scale`.
LK_API int lk_embed_q(int fmt, const int* tokens, const void* codes, long long c_ld, const void* scales, long long s_ld,
                      void* out, int T, int H, int vocab, float scale, void* stream) {
  if (T <= 0) return LKH_OK;
  if (!tokens || !codes || !scales || !out || (H & 31) || ((fmt == GV_W8G16 || fmt == GV_W4) && (H & 255))) return LKH_BAD_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const uint8_t* c = reinterpret_cast<const uint8_t*>(codes);
  const uint8_t* s = reinterpret_cast<const uint8_t*>(scales);
  __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out);
  switch (fmt) {
    case GV_W8: embed_q_kernel<GV_W8><<<T, 128, 0, st>>>(tokens, c, c_ld, s, s_ld, o, H, vocab, scale); break;
    case GV_W8G16: embed_q_kernel<GV_W8G16><<<T, 128, 0, st>>>(tokens, c, c_ld, s, s_ld, o, H, vocab, scale); break;
    case GV_W4: embed_q_kernel<GV_W4><<<T, 128, 0, st>>>(tokens, c, c_ld, s, s_ld, o, H, vocab, scale); break;
    default: return LKH_BAD_ARG;
  }
  lkh::count_launch();
  return lkh::launch_status();
}

// Measurement hook: 0 keeps every GEMV on the register form, 1 (the default) lets the streaming form take
// the shapes it can, 3 the same with L2 hints for the rows the ring does not hold yet.
LK_API void lk_gemv_q_stream(int on) { g_gemv_stream = on; }

// `status` (device word, may be null: then the register form runs) receives the code of a wait that gave up.
// x [M <= 8, K] bf16 (row pitch ldx elements), W as device planes of format `fmt` (1 Q8_0, 2 Q6_K, 3 Q4_K),
// out [M, N] bf16 or, with out_fp32, f32 (row pitch ldo elements).  K a multiple of 32 (256 for the K formats).
LK_API int lk_gemv_q(int fmt, const void* codes, long long c_ld, const void* scales, long long s_ld, const void* x,
                     long long ldx, int M, int N, int K, const float* bias, void* out, long long ldo, int out_fp32,
                     const LkGemvPre* pre, int* status, void* stream) {
  if (M <= 0 || N <= 0) return LKH_OK;
  if (M > 8 || !codes || !scales || !x || !out || (K & 31) || (ldx & 7)) return LKH_BAD_ARG;
  if ((fmt == GV_W8G16 || fmt == GV_W4) && (K & 255)) return LKH_BAD_ARG;
  if (fmt == GV_W4G && ((K & 127) || (s_ld & 3) || (reinterpret_cast<uintptr_t>(scales) & 3))) return LKH_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(codes) & 15) || (c_ld & 15) || (reinterpret_cast<uintptr_t>(x) & 15)) return LKH_BAD_ARG;
  GvParams p;
  p.codes = reinterpret_cast<const uint8_t*>(codes);
  p.scales = reinterpret_cast<const uint8_t*>(scales);
  p.c_ld = c_ld;
  p.s_ld = s_ld;
  p.x = reinterpret_cast<const __nv_bfloat16*>(x);
  p.ldx = ldx;
  p.bias = bias;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.ldo = ldo;
  p.out_fp32 = out_fp32;
  p.M = M;
  p.N = N;
  p.K = K;
  p.slot_expert = nullptr;
  p.slots = p.slot_x_div = p.slot_e_lo = p.slot_e_cnt = 0;
  memset(&p.pre, 0, sizeof(p.pre));
  if (pre) {
    p.pre = *pre;
    if (p.pre.mode < 0 || p.pre.mode > 2 || (p.pre.mode == 1 && !p.pre.gamma)) return LKH_BAD_ARG;
    if (p.pre.mode == 1 && p.pre.delta && ((reinterpret_cast<uintptr_t>(p.pre.delta) & 15) || (p.pre.ldd & 7)))
      return LKH_BAD_ARG;
    if (p.pre.mode == 1 && (reinterpret_cast<uintptr_t>(p.pre.gamma) & 15)) return LKH_BAD_ARG;
    if (p.pre.upd_x) {
      // the update is applied while this kernel's own rows are read: they must be other memory
      if (!p.pre.upd_delta || p.pre.upd_x == x || (p.pre.upd_cols & 7) || (p.pre.upd_ldx & 7) || (p.pre.upd_ldd & 7) ||
          (reinterpret_cast<uintptr_t>(p.pre.upd_x) & 15) || (reinterpret_cast<uintptr_t>(p.pre.upd_delta) & 15))
        return LKH_BAD_ARG;
    }
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int rc;
  switch (fmt) {
    case GV_W8: rc = dispatch_gv<GV_W8>(p, M, st, status); break;
    case GV_W8G16: rc = dispatch_gv<GV_W8G16>(p, M, st, status); break;
    case GV_W4: rc = dispatch_gv<GV_W4>(p, M, st, status); break;
    case GV_W4G: rc = dispatch_gv<GV_W4G>(p, M, st, status); break;
    default: return LKH_BAD_ARG;
  }
  if (rc) return rc;
  lkh::count_launch();
  return lkh::launch_status();
}

// Expert slots: a stack of `n_experts` [N, K] matrices in contiguous planes; slot s multiplies row s / x_div of x
// (bf16, row pitch ldx; with the gated unit in front: 2K wide) by the matrix of expert slot_expert[s] - e_lo (a slot
// whose expert is not in [e_lo, e_lo + n_experts) writes nothing) and writes row s of out [slots, N] (+ bias
// [n_experts, N]).  The expert ids are read on the device, so a routing kernel can come right before this one.
// dry != 0: launch nothing, return 0 if the shape is taken and LKH_BAD_ARG if not.
LK_API int lk_gemv_q_slots(int fmt, const void* codes, const void* scales, const void* x, long long ldx, int slots,
                           int x_div, const int* slot_expert, int e_lo, int n_experts, int N, int K, const float* bias,
                           void* out, long long ldo, const LkGemvPre* pre, int* status, int dry, void* stream) {
  if (slots <= 0 || N <= 0) return LKH_OK;
  if ((K & 31) || ((fmt == GV_W8G16 || fmt == GV_W4) && (K & 255)) || x_div <= 0 || n_experts <= 0) return LKH_BAD_ARG;
  if (!dry && (!codes || !scales || !x || !out || !slot_expert || !status || (ldx & 7) ||
               (reinterpret_cast<uintptr_t>(codes) & 15) || (reinterpret_cast<uintptr_t>(x) & 15)))
    return LKH_BAD_ARG;
  GvParams p;
  memset(&p, 0, sizeof(p));
  p.codes = reinterpret_cast<const uint8_t*>(codes);
  p.scales = reinterpret_cast<const uint8_t*>(scales);
  p.x = reinterpret_cast<const __nv_bfloat16*>(x);
  p.ldx = ldx;
  p.bias = bias;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.ldo = ldo;
  p.M = 1;
  p.N = N;
  p.K = K;
  static const int dummy = 0;
  p.slot_expert = dry ? &dummy : slot_expert;
  p.slots = slots;
  p.slot_x_div = x_div;
  p.slot_e_lo = e_lo;
  p.slot_e_cnt = n_experts;
  if (pre) {
    p.pre = *pre;
    if (p.pre.mode != 0 && p.pre.mode != 2) return LKH_BAD_ARG;       // a norm in front would need the row's own update
    if (p.pre.upd_x) return LKH_BAD_ARG;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  bool taken = false;
  int rc;
  switch (fmt) {
    case GV_W8: p.c_ld = K; p.s_ld = gs_scale_bytes<GV_W8>(K); rc = launch_gs<GV_W8, 1>(p, st, status, &taken, dry != 0); break;
    case GV_W8G16: p.c_ld = K; p.s_ld = gs_scale_bytes<GV_W8G16>(K); rc = launch_gs<GV_W8G16, 1>(p, st, status, &taken, dry != 0); break;
    case GV_W4: p.c_ld = K / 2; p.s_ld = gs_scale_bytes<GV_W4>(K); rc = launch_gs<GV_W4, 1>(p, st, status, &taken, dry != 0); break;
    default: return LKH_BAD_ARG;
  }
  if (rc) return rc;
  if (!taken) return LKH_BAD_ARG;
  if (dry) return LKH_OK;
  lkh::count_launch();
  return lkh::launch_status();
}
