// One kernel per row-parallel layer boundary of a tensor-parallel decoder:
//
//     partial sums of this rank  ->  reduce-scatter  ->  residual add  ->  RMSNorm  ->
//     (e4m3 quantise)  ->  all-gather of the normalised rows
//
// The residual stream stays sharded by rows between the two row-parallel layers (sequence
// parallelism): row r of the step belongs to rank r / ceil(T / world); only that rank adds the
// summed update into its residual row and normalises it, and what travels back is the next
// GEMM's input (one byte per value when it is quantised), not the bf16 sum.
//
// Transport: plain peer stores over NVLink / NVSwitch into the symmetric heap, in a
// "flag-in-data" format: every 16-byte store carries 8 bytes of payload and two copies of the
// collective's epoch number ({d0, epoch, d1, epoch}; the two 8-byte halves may land separately,
// each carries its own flag).  A reader polls the payload itself, so no fence or separate flag
// round trip sits between the data and its consumer: one hop costs one NVLink crossing.  The
// price is twice the bytes, which at decode sizes (<= a few MB) is cheaper than the ~2 us a
// system-scope release costs.  Regions alternate between two halves by epoch parity, like the
// other collectives of symm.cu, so a rank that runs ahead never overwrites what a peer still reads.
//
// One CTA per row.  Phases, in this order in every CTA so that no wait can depend on a later
// phase of a peer: (A) rows owned by a peer: send my partial row to its owner; (B) rows I own:
// wait for the peers' partial rows, sum in rank order, add the residual, normalise, store
// locally and send the result to every peer; (C) rows owned by a peer: wait for the owner's
// result and unpack it into the local output.  Every poll is bounded by the SM clock and reports
// LK_ERR_PEER_TIMEOUT through the status word.  No TMA, no multicast, no multimem.
//
// The reference sums F32 rows with ncclAllReduce and then runs add + RMSNorm as separate
// launches on every card over every row (src/inference/generic_transformer/tp_forward.rs:70-128,
// mod.rs:1063-1101).
#include "common.cuh"
#include "host_common.h"
#include "loken_cuda.h"
#include "symm.cuh"

using namespace lk;

namespace {

constexpr int MAX_CHUNKS = 256 * 8;      // 8 chunks x 256 threads x 8 values = 16384 columns at most

struct TpNormParams {
  SymmView sv;
  const __nv_bfloat16* partial;   // [T, H] this rank's partial sums
  long long ld_p;
  __nv_bfloat16* x;               // [T, H] residual stream; rows this rank owns are updated
  long long ld_x;
  const float* w;                 // [H] norm weight
  float eps;
  int T, H;
  __nv_bfloat16* out_bf16;        // [T, H] normalised rows (all T on every rank), or null
  long long ld_o;
  uint8_t* out_fp8;               // [T, H] e4m3, or null
  float* scales_t;                // [H / 128, scale_ld]
  long long scale_ld;
  int gather;                     // 0: the normalised rows stay on their owner (no phase C)
  int local;                      // 1: `partial` is already the whole update of the owned rows (no phase A)
  int* status;
};

__device__ __forceinline__ void st_ll16(void* p, uint32_t d0, uint32_t d1, uint32_t flag) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(d0), "r"(flag), "r"(d1), "r"(flag)
               : "memory");
}
__device__ __forceinline__ void st_ll8(void* p, uint32_t d0, uint32_t flag) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(d0), "r"(flag) : "memory");
}
__device__ __forceinline__ uint4 ld_ll16(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ uint2 ld_ll8(const void* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}

// `ab` (below) is the CTA's abort word: once one thread has given up on a wait, the others stop waiting
// too (their results are garbage; the status word says so).
__device__ __forceinline__ void add_bf16x2(uint32_t w, float& a, float& b) {
  const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
  a += f.x;
  b += f.y;
}

// Byte layout of one half of the flag-in-data area (the same on every rank):
//   [0, sv.ll_hop2_off)   partial rows on their owner: [source rank][local row][H * 4 bytes]
//   [sv.ll_hop2_off, ..)  results: [row][row_bytes], row_bytes = payload * 2 (+ H / 128 scale words of 8 bytes)
__device__ __forceinline__ long long hop2_row_bytes(int H, bool f8) {
  const long long data = f8 ? (long long)H * 2 : (long long)H * 4;
  const long long sc = f8 ? (long long)(H >> 7) * 8 : 0;
  return (data + sc + 15) & ~15ll;
}

__device__ __forceinline__ bool ll_ok(const uint4& v, unsigned epoch) { return v.y == epoch && v.w == epoch; }

// One bounded step of a batched poll: called when some word of the batch was not valid yet.  Returns
// false when the wait is over (a thread of the CTA gave up, or this one ran out of time).
__device__ __forceinline__ bool poll_again(unsigned& spins, long long& t0, volatile int* ab, int* status, int src) {
  if (spins == 0) t0 = clock64();
  if ((++spins & 15u) == 0u) {
    if (*ab) return false;
    if (clock64() - t0 > LK_PEER_WAIT_CYCLES) {
      *ab = 1;
      if (status) atomicCAS(status, 0, LK_ERR_PEER_TIMEOUT | (src << 8));
      return false;
    }
  }
  return true;
}

// NT threads per CTA, IT chunks of eight values per thread: NT * IT * 8 >= H.  Every wait is a batched
// poll: all the words a thread needs in a step are requested together, and the ones that have not
// arrived are requested again together, so a late peer costs one round trip per retry, not one per word.
template <int W, int NT, int IT>
__global__ void __launch_bounds__(NT)
tp_sum_norm_kernel(const TpNormParams p) {
  pdl_wait();
  pdl_launch();
  __shared__ float red[32];
  __shared__ int s_abort;
  if (threadIdx.x == 0) s_abort = 0;
  __syncthreads();
  volatile int* ab = &s_abort;
  const int me = p.sv.rank;
  const int T = p.T, H = p.H;
  const int rpr = (T + W - 1) / W;          // rows per rank
  const unsigned epoch = symm_epoch_begin(p.sv);
  const int half = epoch & 1;
  const long long half_off = p.sv.ll_off + (long long)half * p.sv.ll_half_bytes;
  const int nchunk = H >> 3;
  const bool f8 = p.out_fp8 != nullptr;
  const long long hop1_row = (long long)H * 4;
  const long long hop2_data = f8 ? (long long)H * 2 : (long long)H * 4;
  const long long hop2_row = hop2_row_bytes(H, f8);

  // ---- phase A: my partial of a row somebody else owns goes to its owner ----
  const bool local = p.local != 0;
  for (int r = blockIdx.x; r < T && !local; r += gridDim.x) {
    const int own = r / rpr;
    if (own == me) continue;
    char* dst = reinterpret_cast<char*>(p.sv.base[own]) + half_off + ((long long)me * rpr + (r - own * rpr)) * hop1_row;
    const __nv_bfloat16* src = p.partial + (long long)r * p.ld_p;
    for (int c = threadIdx.x; c < nchunk; c += NT) {
      const uint4 q = *reinterpret_cast<const uint4*>(src + c * 8);
      st_ll16(dst + (long long)c * 32, q.x, q.y, epoch);
      st_ll16(dst + (long long)c * 32 + 16, q.z, q.w, epoch);
    }
  }

  // ---- phase B: rows I own ----
  const char* mine = reinterpret_cast<const char*>(p.sv.base[me]) + half_off;
  for (int r = blockIdx.x; r < T; r += gridDim.x) {
    if (r / rpr != me) continue;
    const int rl = r - me * rpr;
    float v[IT][8];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < IT; ++it) {
      const int c = it * NT + threadIdx.x;
      if (c < nchunk) {
        uint4 q[W][2];
        const uint4 own_q = *reinterpret_cast<const uint4*>(p.partial + (long long)r * p.ld_p + c * 8);
        if (!local) {
          const char* src0 = mine + (long long)rl * hop1_row + (long long)c * 32;
          const long long sstep = (long long)rpr * hop1_row;
#pragma unroll
          for (int s = 0; s < W; ++s) {
            if (s != me) {
              q[s][0] = ld_ll16(src0 + s * sstep);
              q[s][1] = ld_ll16(src0 + s * sstep + 16);
            }
          }
          unsigned spins = 0;
          long long t0 = 0;
          while (true) {
            bool all = true;
            int late = 0;
#pragma unroll
            for (int s = 0; s < W; ++s)
              if (s != me && !(ll_ok(q[s][0], epoch) && ll_ok(q[s][1], epoch))) {
                all = false;
                late = s;
              }
            if (all || !poll_again(spins, t0, ab, p.status, late)) break;
#pragma unroll
            for (int s = 0; s < W; ++s) {
              if (s != me) {
                if (!ll_ok(q[s][0], epoch)) q[s][0] = ld_ll16(src0 + s * sstep);
                if (!ll_ok(q[s][1], epoch)) q[s][1] = ld_ll16(src0 + s * sstep + 16);
              }
            }
          }
        }
        float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int s = 0; s < W; ++s) {       // rank order: the same bits whichever peer arrives first
          if (s == me) {
            add_bf16x2(own_q.x, a[0], a[1]);
            add_bf16x2(own_q.y, a[2], a[3]);
            add_bf16x2(own_q.z, a[4], a[5]);
            add_bf16x2(own_q.w, a[6], a[7]);
          } else if (!local) {
            add_bf16x2(q[s][0].x, a[0], a[1]);
            add_bf16x2(q[s][0].z, a[2], a[3]);
            add_bf16x2(q[s][1].x, a[4], a[5]);
            add_bf16x2(q[s][1].z, a[6], a[7]);
          }
        }
        __nv_bfloat16* xr = p.x + (long long)r * p.ld_x + c * 8;
        const uint4 xq = *reinterpret_cast<const uint4*>(xr);
        add_bf16x2(xq.x, a[0], a[1]);
        add_bf16x2(xq.y, a[2], a[3]);
        add_bf16x2(xq.z, a[4], a[5]);
        add_bf16x2(xq.w, a[6], a[7]);
        // the residual stream is bf16: round once, then normalise what was stored
        uint4 xo;
        __nv_bfloat162* xo2 = reinterpret_cast<__nv_bfloat162*>(&xo);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          xo2[e] = __floats2bfloat162_rn(a[2 * e], a[2 * e + 1]);
          const float2 f = __bfloat1622float2(xo2[e]);
          v[it][2 * e] = f.x;
          v[it][2 * e + 1] = f.y;
          ss += f.x * f.x + f.y * f.y;
        }
        *reinterpret_cast<uint4*>(xr) = xo;
      }
    }
    ss = block_sum(ss, red);
    const float rinv = rsqrtf(ss / (float)H + p.eps);
#pragma unroll
    for (int it = 0; it < IT; ++it) {
      const int c = it * NT + threadIdx.x;
      if (c < nchunk) {
        const float4* w4 = reinterpret_cast<const float4*>(p.w + c * 8);
        const float4 wa = w4[0], wb = w4[1];
        float o[8] = {v[it][0] * rinv * wa.x, v[it][1] * rinv * wa.y, v[it][2] * rinv * wa.z, v[it][3] * rinv * wa.w,
                      v[it][4] * rinv * wb.x, v[it][5] * rinv * wb.y, v[it][6] * rinv * wb.z, v[it][7] * rinv * wb.w};
        uint4 ob;
        __nv_bfloat162* ob2 = reinterpret_cast<__nv_bfloat162*>(&ob);
#pragma unroll
        for (int e = 0; e < 4; ++e) ob2[e] = __floats2bfloat162_rn(o[2 * e], o[2 * e + 1]);
        if (p.out_bf16) *reinterpret_cast<uint4*>(p.out_bf16 + (long long)r * p.ld_o + c * 8) = ob;
        if (f8) {
          // quantise what a bf16 consumer would have seen; the 16 threads of a 128-group agree on amax
          float amax = 0.f;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(ob2[e]);
            o[2 * e] = f.x;
            o[2 * e + 1] = f.y;
            amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
          }
          const unsigned hm = 0xFFFFu << (threadIdx.x & 16);
#pragma unroll
          for (int s = 8; s > 0; s >>= 1) amax = fmaxf(amax, __shfl_xor_sync(hm, amax, s));
          const float scale = e4m3_group_scale(amax);
          const float inv = 1.f / scale;
          uint2 q8;
          uint8_t* b = reinterpret_cast<uint8_t*>(&q8);
#pragma unroll
          for (int e = 0; e < 8; ++e) b[e] = f2e4m3(o[e] * inv);
          *reinterpret_cast<uint2*>(p.out_fp8 + (long long)r * H + c * 8) = q8;
          const bool writer = (threadIdx.x & 15) == 0;
          if (writer) p.scales_t[(long long)(c >> 4) * p.scale_ld + r] = scale;
          if (p.gather) {
#pragma unroll
            for (int d = 1; d < W; ++d) {
              char* dst = reinterpret_cast<char*>(p.sv.base[(me + d) % W]) + half_off + p.sv.ll_hop2_off +
                          (long long)r * hop2_row;
              st_ll16(dst + (long long)c * 16, q8.x, q8.y, epoch);
              if (writer) st_ll8(dst + hop2_data + (long long)(c >> 4) * 8, __float_as_uint(scale), epoch);
            }
          }
        } else if (p.gather) {
#pragma unroll
          for (int d = 1; d < W; ++d) {
            char* dst = reinterpret_cast<char*>(p.sv.base[(me + d) % W]) + half_off + p.sv.ll_hop2_off +
                        (long long)r * hop2_row;
            st_ll16(dst + (long long)c * 32, ob.x, ob.y, epoch);
            st_ll16(dst + (long long)c * 32 + 16, ob.z, ob.w, epoch);
          }
        }
      }
    }
    __syncthreads();      // `red` is reused by the next owned row
  }

  // ---- phase C: the owners' results for the other rows ----
  if (p.gather) {
    for (int r = blockIdx.x; r < T; r += gridDim.x) {
      const int own = r / rpr;
      if (own == me) continue;
      const char* src = mine + p.sv.ll_hop2_off + (long long)r * hop2_row;
      if (f8) {
        // a thread's IT payload words and (the first H / 128 threads) one scale word, all in one batch
        uint4 a[IT];
        const bool has_sc = threadIdx.x < (H >> 7);
        uint2 sc = make_uint2(0u, epoch);
#pragma unroll
        for (int it = 0; it < IT; ++it) {
          const int c = it * NT + threadIdx.x;
          a[it] = c < nchunk ? ld_ll16(src + (long long)c * 16) : make_uint4(0u, epoch, 0u, epoch);
        }
        if (has_sc) sc = ld_ll8(src + hop2_data + (long long)threadIdx.x * 8);
        unsigned spins = 0;
        long long t0 = 0;
        while (true) {
          bool all = sc.y == epoch;
#pragma unroll
          for (int it = 0; it < IT; ++it) all = all && ll_ok(a[it], epoch);
          if (all || !poll_again(spins, t0, ab, p.status, own)) break;
#pragma unroll
          for (int it = 0; it < IT; ++it)
            if (!ll_ok(a[it], epoch)) a[it] = ld_ll16(src + (long long)(it * NT + threadIdx.x) * 16);
          if (sc.y != epoch) sc = ld_ll8(src + hop2_data + (long long)threadIdx.x * 8);
        }
#pragma unroll
        for (int it = 0; it < IT; ++it) {
          const int c = it * NT + threadIdx.x;
          if (c < nchunk) *reinterpret_cast<uint2*>(p.out_fp8 + (long long)r * H + c * 8) = make_uint2(a[it].x, a[it].z);
        }
        if (has_sc) p.scales_t[(long long)threadIdx.x * p.scale_ld + r] = __uint_as_float(sc.x);
      } else {
        uint4 a[IT][2];
#pragma unroll
        for (int it = 0; it < IT; ++it) {
          const int c = it * NT + threadIdx.x;
          if (c < nchunk) {
            a[it][0] = ld_ll16(src + (long long)c * 32);
            a[it][1] = ld_ll16(src + (long long)c * 32 + 16);
          } else {
            a[it][0] = a[it][1] = make_uint4(0u, epoch, 0u, epoch);
          }
        }
        unsigned spins = 0;
        long long t0 = 0;
        while (true) {
          bool all = true;
#pragma unroll
          for (int it = 0; it < IT; ++it) all = all && ll_ok(a[it][0], epoch) && ll_ok(a[it][1], epoch);
          if (all || !poll_again(spins, t0, ab, p.status, own)) break;
#pragma unroll
          for (int it = 0; it < IT; ++it) {
            const long long off = (long long)(it * NT + threadIdx.x) * 32;
            if (!ll_ok(a[it][0], epoch)) a[it][0] = ld_ll16(src + off);
            if (!ll_ok(a[it][1], epoch)) a[it][1] = ld_ll16(src + off + 16);
          }
        }
#pragma unroll
        for (int it = 0; it < IT; ++it) {
          const int c = it * NT + threadIdx.x;
          if (c < nchunk)
            *reinterpret_cast<uint4*>(p.out_bf16 + (long long)r * p.ld_o + c * 8) =
                make_uint4(a[it][0].x, a[it][0].z, a[it][1].x, a[it][1].z);
        }
      }
    }
  }
  symm_epoch_end(p.sv);
}

template <int W>
void launch_sum_norm(const TpNormParams& p, int grid, cudaStream_t st) {
  const int nchunk = p.H >> 3;
  // more ranks mean more words per chunk in flight: more threads with fewer chunks each keep the
  // sequential steps of an owned row few
  if (W >= 4 && nchunk <= 512 * 2)
    lkh::launch_pdl(tp_sum_norm_kernel<W, 512, 2>, dim3(grid), dim3(512), 0, st, p);
  else if (nchunk <= 256 * 4)
    lkh::launch_pdl(tp_sum_norm_kernel<W, 256, 4>, dim3(grid), dim3(256), 0, st, p);
  else
    lkh::launch_pdl(tp_sum_norm_kernel<W, 256, 8>, dim3(grid), dim3(256), 0, st, p);
}

}  // namespace

// Sum of the ranks' partial rows + residual + RMSNorm (+ e4m3 quantise), rows sharded over the
// ranks in between.  `x` rows owned by this rank (row r belongs to rank r / ceil(T / world)) are
// updated in place; `out_bf16` / `out_fp8` + `scales_t` receive the normalised rows: all T of them
// when `gather` is set, only the owned ones otherwise.
LK_API int lk_tp_sum_norm(const void* view, const void* partial, long long ld_p, void* x, long long ld_x,
                          const float* w, float eps, int T, int H, void* out_bf16, long long ld_o, void* out_fp8,
                          float* scales_t, long long scale_ld, int gather, int local, int* status, void* stream) {
  if (!view || !partial || !x || !w || (!out_bf16 && !out_fp8)) return LKH_BAD_ARG;
  if (T <= 0) return LKH_OK;
  TpNormParams p;
  p.sv = *reinterpret_cast<const SymmView*>(view);
  const int W = p.sv.world;
  if (H % 8 || (out_fp8 && (H % 128 || !scales_t)) || (H >> 3) > MAX_CHUNKS) return LKH_BAD_ARG;
  if ((ld_p & 7) || (ld_x & 7) || (out_bf16 && (ld_o & 7))) return LKH_BAD_ARG;
  if (out_bf16 && out_fp8 && gather) return LKH_BAD_ARG;      // one payload format per call travels
  const long long rpr = (T + W - 1) / W;
  const bool f8 = out_fp8 != nullptr;
  const long long row2 = (((f8 ? (long long)H * 2 + (long long)(H >> 7) * 8 : (long long)H * 4)) + 15) & ~15ll;
  if (p.sv.ll_half_bytes <= 0 || (long long)W * rpr * H * 4 > p.sv.ll_hop2_off ||
      p.sv.ll_hop2_off + (long long)T * row2 > p.sv.ll_half_bytes)
    return LKH_TOO_LARGE;
  p.partial = reinterpret_cast<const __nv_bfloat16*>(partial);
  p.ld_p = ld_p;
  p.x = reinterpret_cast<__nv_bfloat16*>(x);
  p.ld_x = ld_x;
  p.w = w;
  p.eps = eps;
  p.T = T;
  p.H = H;
  p.out_bf16 = reinterpret_cast<__nv_bfloat16*>(out_bf16);
  p.ld_o = ld_o;
  p.out_fp8 = reinterpret_cast<uint8_t*>(out_fp8);
  p.scales_t = scales_t;
  p.scale_ld = scale_ld;
  p.gather = gather;
  p.local = local;
  p.status = status;
  const int grid = T < 148 ? T : 148;        // every CTA waits on peers: all of them resident at once
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (W) {
    case 1: launch_sum_norm<1>(p, grid, st); break;
    case 2: launch_sum_norm<2>(p, grid, st); break;
    case 4: launch_sum_norm<4>(p, grid, st); break;
    case 8: launch_sum_norm<8>(p, grid, st); break;
    default: return LKH_BAD_ARG;
  }
  lkh::count_launch();
  return lkh::launch_status();
}
