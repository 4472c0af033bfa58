// Expert-parallel token dispatch and combine over peer memory (all-to-all without a host round
// trip), for a residual stream that is sharded by rows over the ranks (tp_fused.cu):
//
//   lk_ep_dispatch   every (token, choice) pair of the rows this rank owns goes to the rank that
//                    holds the chosen expert: the normalised hidden row plus (expert id, token,
//                    choice) lands in that rank's slot region [source rank][position]; positions
//                    are the pair's rank among earlier pairs with the same destination, so the
//                    layout is deterministic; a count per destination goes along
//   lk_ep_meta       receiver: waits for every source's count and the metadata of its pairs,
//                    writes the expert id of every slot (-1 for unused slots) for lk_moe_plan
//   lk_ep_gather     receiver: unpacks the arrived rows into a dense bf16 buffer, one row per slot;
//                    the grouped expert GEMMs then run over them as over local pairs
//   lk_ep_return     receiver: each slot's expert output row goes back to its source rank at
//                    [token][choice]
//   lk_ep_combine    owner: waits for the k rows of each of its tokens and sums them in choice order
//                    with the router weights in fp32 (the same fold order at every degree)
//
// Transport is the flag-in-data format of tp_fused.cu ({d0, epoch, d1, epoch} per 16-byte store):
// readers poll the payload, nothing fences.  Dispatch (three kernels) is one collective with one
// epoch, ended by lk_ep_gather; return + combine is the next, ended by lk_ep_combine.  Plain peer
// stores only: no TMA, no multicast, no multimem.  Every poll is bounded and reports
// LK_ERR_PEER_TIMEOUT through the status word.
//
// The reference has no all-to-all: it copies every row to every shard card, zero-weights foreign
// pairs and sums the partial products (src/inference/generic_transformer/moe_weights.rs:1779-1893,
// cuda/moe/tp_local.cu:14-57); its fold order is the router's slot order (cuda/moe/moe_mmq.cu:12-14).
#include "common.cuh"
#include "host_common.h"
#include "loken_cuda.h"
#include "symm.cuh"

using namespace lk;

namespace {

constexpr int EP_NT = 128;
constexpr int EP_HDR = 256;        // bytes reserved for the per-source counts at the start of a half

__device__ __forceinline__ void st_ll16(void* p, uint32_t d0, uint32_t d1, uint32_t flag) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(d0), "r"(flag), "r"(d1), "r"(flag)
               : "memory");
}
__device__ __forceinline__ uint4 ld_ll16(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ bool ll_wait16(const void* p, unsigned epoch, uint4& v, volatile int* ab, int* status,
                                          int src) {
  v = ld_ll16(p);
  if (v.y == epoch && v.w == epoch) return true;
  const long long t0 = clock64();
  for (unsigned it = 1;; ++it) {
    v = ld_ll16(p);
    if (v.y == epoch && v.w == epoch) return true;
    if ((it & 63u) == 0u) {
      if (*ab) return false;
      if (clock64() - t0 > LK_PEER_WAIT_CYCLES) break;
    }
  }
  *ab = 1;
  if (status) atomicCAS(status, 0, LK_ERR_PEER_TIMEOUT | (src << 8));
  return false;
}

struct EpGeom {
  int T, H, k, world, me;
  int rpr;          // rows per rank
  int cap;          // slots per source on a receiver = rpr * k
  int epr;          // experts per rank
  long long slot_bytes;   // 16 (metadata) + 4 * H (row payload, flag-in-data)
};
__device__ __host__ __forceinline__ EpGeom ep_geom(const SymmView& sv, int T, int H, int k, int n_experts) {
  EpGeom g;
  g.T = T; g.H = H; g.k = k; g.world = sv.world; g.me = sv.rank;
  g.rpr = (T + sv.world - 1) / sv.world;
  g.cap = g.rpr * k;
  g.epr = n_experts / sv.world;
  g.slot_bytes = 16 + (long long)H * 4;
  return g;
}

// ---- dispatch ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(EP_NT)
ep_dispatch_kernel(const SymmView sv, const __nv_bfloat16* __restrict__ h, long long ldh, const int* __restrict__ ids,
                   int T, int H, int k, int n_experts, int* __restrict__ status) {
  pdl_wait();
  pdl_launch();
  __shared__ int red[EP_NT / 32];
  const EpGeom g = ep_geom(sv, T, H, k, n_experts);
  const int lo = min(T, g.me * g.rpr), hi = min(T, lo + g.rpr);
  const int n_pairs = (hi - lo) * k;
  const unsigned epoch = symm_epoch_begin(sv);
  const long long half_off = sv.ll_off + (long long)(epoch & 1) * sv.ll_half_bytes;
  const int p = blockIdx.x;
  if (p == 0 && threadIdx.x < g.world) {
    // how many of my pairs each destination gets
    int c = 0;
    for (int q = 0; q < n_pairs; ++q) {
      const int e = ids[q];
      c += (e >= 0 && e < n_experts && e / g.epr == (int)threadIdx.x) ? 1 : 0;
    }
    char* dst = reinterpret_cast<char*>(sv.base[threadIdx.x]) + half_off + g.me * 16;
    st_ll16(dst, (uint32_t)c, 0u, epoch);
  }
  if (p >= n_pairs) return;
  const int e = ids[p];
  if (e < 0 || e >= n_experts) {
    if (threadIdx.x == 0 && status) atomicCAS(status, 0, LK_ERR_BOUNDS | (7 << 8));
    return;
  }
  const int dest = e / g.epr;
  // position among my earlier pairs with the same destination
  int c = 0;
  for (int q = threadIdx.x; q < p; q += EP_NT) {
    const int eq = ids[q];
    c += (eq >= 0 && eq < n_experts && eq / g.epr == dest) ? 1 : 0;
  }
  c = (int)warp_sum((float)c);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = c;
  __syncthreads();
  int pos = 0;
#pragma unroll
  for (int w = 0; w < EP_NT / 32; ++w) pos += red[w];
  const int t_local = p / k, j = p - t_local * k;
  char* dst = reinterpret_cast<char*>(sv.base[dest]) + half_off + EP_HDR + ((long long)g.me * g.cap + pos) * g.slot_bytes;
  if (threadIdx.x == 0) st_ll16(dst, (uint32_t)e, (uint32_t)((t_local << 8) | j), epoch);
  const __nv_bfloat16* src = h + (long long)(lo + t_local) * ldh;
  for (int cch = threadIdx.x; cch < (H >> 3); cch += EP_NT) {
    const uint4 q = *reinterpret_cast<const uint4*>(src + cch * 8);
    st_ll16(dst + 16 + (long long)cch * 32, q.x, q.y, epoch);
    st_ll16(dst + 32 + (long long)cch * 32, q.z, q.w, epoch);
  }
}

// ---- receiver: counts + metadata -> expert id per slot ----------------------------------------------
__global__ void __launch_bounds__(256)
ep_meta_kernel(const SymmView sv, int T, int H, int k, int n_experts, int* __restrict__ slot_expert,
               int* __restrict__ slot_src, int* __restrict__ status) {
  pdl_wait();
  pdl_launch();
  __shared__ int cnt[MAX_RANKS];
  __shared__ int s_abort;
  if (threadIdx.x == 0) s_abort = 0;
  __syncthreads();
  volatile int* ab = &s_abort;
  const EpGeom g = ep_geom(sv, T, H, k, n_experts);
  const unsigned epoch = symm_epoch_begin(sv);
  const char* mine = reinterpret_cast<const char*>(sv.base[g.me]) + sv.ll_off + (long long)(epoch & 1) * sv.ll_half_bytes;
  if (threadIdx.x < g.world) {
    uint4 v;
    const bool ok = ll_wait16(mine + threadIdx.x * 16, epoch, v, ab, status, threadIdx.x);
    int c = ok ? (int)v.x : 0;
    if (c < 0 || c > g.cap) {
      if (status) atomicCAS(status, 0, LK_ERR_BOUNDS | (8 << 8));
      c = 0;
    }
    cnt[threadIdx.x] = c;
  }
  __syncthreads();
  const int slots = g.world * g.cap;
  for (int i = threadIdx.x; i < slots; i += blockDim.x) {
    const int s = i / g.cap, q = i - s * g.cap;
    int e = -1, info = 0;
    if (q < cnt[s]) {
      uint4 v;
      if (ll_wait16(mine + EP_HDR + (long long)i * g.slot_bytes, epoch, v, ab, status, s)) {
        e = (int)v.x;
        info = (s << 24) | (int)(v.z & 0xFFFFFF);
      }
    }
    slot_expert[i] = e;
    slot_src[i] = info;
  }
}

// ---- receiver: arrived rows -> dense bf16 rows, one per slot -----------------------------------------
__global__ void __launch_bounds__(EP_NT)
ep_gather_kernel(const SymmView sv, int T, int H, int k, int n_experts, const int* __restrict__ slot_expert,
                 __nv_bfloat16* __restrict__ xr, long long ldx, int* __restrict__ status) {
  pdl_wait();
  pdl_launch();
  __shared__ int s_abort;
  if (threadIdx.x == 0) s_abort = 0;
  __syncthreads();
  volatile int* ab = &s_abort;
  const EpGeom g = ep_geom(sv, T, H, k, n_experts);
  const unsigned epoch = symm_epoch_begin(sv);
  const char* mine = reinterpret_cast<const char*>(sv.base[g.me]) + sv.ll_off + (long long)(epoch & 1) * sv.ll_half_bytes;
  const int slots = g.world * g.cap;
  for (int i = blockIdx.x; i < slots; i += gridDim.x) {
    if (slot_expert[i] < 0) continue;
    const char* src = mine + EP_HDR + (long long)i * g.slot_bytes + 16;
    __nv_bfloat16* dst = xr + (long long)i * ldx;
    for (int c = threadIdx.x; c < (H >> 3); c += EP_NT) {
      uint4 a = ld_ll16(src + (long long)c * 32), b = ld_ll16(src + (long long)c * 32 + 16);
      if (!(a.y == epoch && a.w == epoch)) ll_wait16(src + (long long)c * 32, epoch, a, ab, status, i / g.cap);
      if (!(b.y == epoch && b.w == epoch)) ll_wait16(src + (long long)c * 32 + 16, epoch, b, ab, status, i / g.cap);
      *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(a.x, a.z, b.x, b.z);
    }
  }
  symm_epoch_end(sv);
}

// ---- receiver: expert outputs back to the owners of their tokens ---------------------------------------
__global__ void __launch_bounds__(EP_NT)
ep_return_kernel(const SymmView sv, int T, int H, int k, int n_experts, const int* __restrict__ slot_src,
                 const int* __restrict__ pair_row, const __nv_bfloat16* __restrict__ y, long long ldy) {
  pdl_wait();
  pdl_launch();
  const EpGeom g = ep_geom(sv, T, H, k, n_experts);
  const unsigned epoch = symm_epoch_begin(sv);
  const long long half_off = sv.ll_off + (long long)(epoch & 1) * sv.ll_half_bytes;
  const int slots = g.world * g.cap;
  for (int i = blockIdx.x; i < slots; i += gridDim.x) {
    const int row = pair_row[i];
    if (row < 0) continue;
    const int info = slot_src[i];
    const int s = (info >> 24) & 0xFF, t_local = (info >> 8) & 0xFFFF, j = info & 0xFF;
    if (s >= g.world || t_local >= g.rpr || j >= k) continue;
    char* dst = reinterpret_cast<char*>(sv.base[s]) + half_off + ((long long)t_local * k + j) * ((long long)H * 4);
    const __nv_bfloat16* src = y + (long long)row * ldy;
    for (int c = threadIdx.x; c < (H >> 3); c += EP_NT) {
      const uint4 q = *reinterpret_cast<const uint4*>(src + c * 8);
      st_ll16(dst + (long long)c * 32, q.x, q.y, epoch);
      st_ll16(dst + (long long)c * 32 + 16, q.z, q.w, epoch);
    }
  }
}

// ---- owner: weighted sum of each token's k rows, in choice order -----------------------------------------
__global__ void __launch_bounds__(EP_NT)
ep_combine_kernel(const SymmView sv, int T, int H, int k, int n_experts, const float* __restrict__ wts,
                  __nv_bfloat16* __restrict__ out, long long ldo, int* __restrict__ status) {
  pdl_wait();
  pdl_launch();
  __shared__ int s_abort;
  if (threadIdx.x == 0) s_abort = 0;
  __syncthreads();
  volatile int* ab = &s_abort;
  const EpGeom g = ep_geom(sv, T, H, k, n_experts);
  const int lo = min(T, g.me * g.rpr), hi = min(T, lo + g.rpr);
  const unsigned epoch = symm_epoch_begin(sv);
  const char* mine = reinterpret_cast<const char*>(sv.base[g.me]) + sv.ll_off + (long long)(epoch & 1) * sv.ll_half_bytes;
  for (int t = blockIdx.x; t < hi - lo; t += gridDim.x) {
    for (int c = threadIdx.x; c < (H >> 3); c += EP_NT) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int j = 0; j < k; ++j) {
        const char* src = mine + ((long long)t * k + j) * ((long long)H * 4) + (long long)c * 32;
        uint4 a = ld_ll16(src), b = ld_ll16(src + 16);
        if (!(a.y == epoch && a.w == epoch)) ll_wait16(src, epoch, a, ab, status, j);
        if (!(b.y == epoch && b.w == epoch)) ll_wait16(src + 16, epoch, b, ab, status, j);
        const float w = wts[(long long)t * k + j];
        const uint32_t ws[4] = {a.x, a.z, b.x, b.z};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ws[e]));
          acc[2 * e] = fmaf(w, f.x, acc[2 * e]);
          acc[2 * e + 1] = fmaf(w, f.y, acc[2 * e + 1]);
        }
      }
      uint4 o;
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e) oh[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
      *reinterpret_cast<uint4*>(out + (long long)(lo + t) * ldo + c * 8) = o;
    }
  }
  symm_epoch_end(sv);
}

int ep_check(const SymmView& sv, int T, int H, int k, int n_experts) {
  if (T <= 0 || (H & 7) || k < 1 || k > 255 || n_experts < sv.world || n_experts % sv.world) return LKH_BAD_ARG;
  const EpGeom g = ep_geom(sv, T, H, k, n_experts);
  if (g.rpr > 65535) return LKH_BAD_ARG;
  const long long need = EP_HDR + (long long)sv.world * g.cap * g.slot_bytes;
  if (sv.ll_half_bytes <= 0 || need > sv.ll_half_bytes) return LKH_TOO_LARGE;
  return LKH_OK;
}

}  // namespace

// Slots a receiver holds for a step of T rows: world * ceil(T / world) * k.
LK_API int lk_ep_slots(const void* view, int T, int k) {
  const SymmView& sv = *reinterpret_cast<const SymmView*>(view);
  return sv.world * ((T + sv.world - 1) / sv.world) * k;
}

// h: normalised hidden rows [T, H] of which this rank's own rows are current; ids: [own rows, k] expert ids.
LK_API int lk_ep_dispatch(const void* view, const void* h, long long ldh, const int* ids, int T, int H, int k,
                          int n_experts, int* status, void* stream) {
  const SymmView& sv = *reinterpret_cast<const SymmView*>(view);
  const int rc = ep_check(sv, T, H, k, n_experts);
  if (rc) return rc;
  const int rpr = (T + sv.world - 1) / sv.world;
  const int lo = T < sv.rank * rpr ? T : sv.rank * rpr, hi = T < lo + rpr ? T : lo + rpr;
  const int n_pairs = (hi - lo) * k;
  lkh::launch_pdl(ep_dispatch_kernel, dim3(n_pairs > 0 ? n_pairs : 1), dim3(EP_NT), 0, (cudaStream_t)stream, sv,
                  (const __nv_bfloat16*)h, ldh, ids, T, H, k, n_experts, status);
  lkh::count_launch();
  return lkh::launch_status();
}

LK_API int lk_ep_meta(const void* view, int T, int H, int k, int n_experts, int* slot_expert, int* slot_src,
                      int* status, void* stream) {
  const SymmView& sv = *reinterpret_cast<const SymmView*>(view);
  const int rc = ep_check(sv, T, H, k, n_experts);
  if (rc) return rc;
  lkh::launch_pdl(ep_meta_kernel, dim3(1), dim3(256), 0, (cudaStream_t)stream, sv, T, H, k, n_experts, slot_expert,
                  slot_src, status);
  lkh::count_launch();
  return lkh::launch_status();
}

LK_API int lk_ep_gather(const void* view, int T, int H, int k, int n_experts, const int* slot_expert, void* xr,
                        long long ldx, int* status, void* stream) {
  const SymmView& sv = *reinterpret_cast<const SymmView*>(view);
  const int rc = ep_check(sv, T, H, k, n_experts);
  if (rc) return rc;
  const int slots = lk_ep_slots(view, T, k);
  lkh::launch_pdl(ep_gather_kernel, dim3(slots < 148 ? slots : 148), dim3(EP_NT), 0, (cudaStream_t)stream, sv, T, H,
                  k, n_experts, slot_expert, (__nv_bfloat16*)xr, ldx, status);
  lkh::count_launch();
  return lkh::launch_status();
}

LK_API int lk_ep_return(const void* view, int T, int H, int k, int n_experts, const int* slot_src,
                        const int* pair_row, const void* y, long long ldy, void* stream) {
  const SymmView& sv = *reinterpret_cast<const SymmView*>(view);
  const int rc = ep_check(sv, T, H, k, n_experts);
  if (rc) return rc;
  const int slots = lk_ep_slots(view, T, k);
  lkh::launch_pdl(ep_return_kernel, dim3(slots < 296 ? slots : 296), dim3(EP_NT), 0, (cudaStream_t)stream, sv, T, H,
                  k, n_experts, slot_src, pair_row, (const __nv_bfloat16*)y, ldy);
  lkh::count_launch();
  return lkh::launch_status();
}

// wts: [own rows, k] router weights; out rows [lo, hi) of [T, H] receive the weighted sums.
LK_API int lk_ep_combine(const void* view, int T, int H, int k, int n_experts, const float* wts, void* out,
                         long long ldo, int* status, void* stream) {
  const SymmView& sv = *reinterpret_cast<const SymmView*>(view);
  const int rc = ep_check(sv, T, H, k, n_experts);
  if (rc) return rc;
  const int rpr = (T + sv.world - 1) / sv.world;
  const int lo = T < sv.rank * rpr ? T : sv.rank * rpr, hi = T < lo + rpr ? T : lo + rpr;
  const int n = hi - lo;
  lkh::launch_pdl(ep_combine_kernel, dim3(n > 0 ? n : 1), dim3(EP_NT), 0, (cudaStream_t)stream, sv, T, H, k,
                  n_experts, wts, (__nv_bfloat16*)out, ldo, status);
  lkh::count_launch();
  return lkh::launch_status();
}
