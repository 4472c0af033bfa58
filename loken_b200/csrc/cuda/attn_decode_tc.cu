// Flash decode over the q8 paged KV cache on the 5th-generation tensor cores
// (head_dim 128, 16-token pages, up to 8 query heads per kv head).
//
// The SIMT decode kernels of this library spend ~80 warp instructions per key on dp4a, int->float
// conversions and FMAs.  Here both products run as tcgen05.mma kind::i8 straight from the pages
// TMA wrote, and the 128 compute threads only do the softmax:
//
//   tile = 128 keys = 8 pages; K and V land in shared memory exactly as stored ([key][128 int8],
//   128-byte swizzle) and are never converted.
//   scores  S^T[key, head] per 32-value block b:  A = K tile (K-major, block b = byte offset 32 b),
//           B = int8 queries [16 x 128] (rows >= G are zero), D = 128 lanes x 16 columns of s32 in
//           TMEM.  Thread t (= key t) reads its lane and folds the per-32 scales:
//           s = sum_b acc_b * dk[t,b] * dq[head,b].
//   values  O^T[dim, head] = V^T (MN-major A: the same bytes, read transposed) times P.  The value
//           scale dv[t,b] belongs to (key, block of the dim), so block b gets its own B operand
//           P_b[t, head] = p[t, head] * dv[t,b] / dvmax_b, as 15-bit fixed point split into a high
//           and a low byte; the two bytes sit in rows g and 8 + g of block b's 16 rows of a 64-row B
//           tile, so one N = 64 MMA per 32 keys yields all eight partial sums.  Rows 32 b .. 32 b + 31 of that MMA's
//           result are the ones that matter; thread d (= dim d) reads columns of block d / 32.
//   online softmax per tile: tile maxima by redux.sync + one shared-memory exchange; the running
//           output lives in registers (8 floats per thread) and is rescaled once per tile.
// Warps 0-3 compute, warp 4 issues TMA, warp 5 issues MMA and owns the TMEM allocation.
// Every wait is bounded; TMA loads are plain (no multicast) and touch only this GPU's memory.
#include "attn_decode_common.cuh"
#include "host_common.h"
#include "loken_cuda.h"

using namespace lk;

namespace {

constexpr int HD = 128;
constexpr int PAGE = 16;
constexpr int TILE = 128;
constexpr int STAGES = 3;
constexpr int STAGE_BYTES = 2 * TILE * HD;       // K tile then V tile, 16 KB each
constexpr int PB_BYTES = 16 * 128;               // one B tile of P (16 rows x 128 keys)
constexpr uint32_t TMEM_COLS = 128;              // S: 4 x 16 columns, O: 4 x 16 columns
constexpr uint32_t IDESC_QK = (2u << 4) | (1u << 7) | (1u << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
// A = int8 read MN-major (bit 15), B = unsigned bytes
constexpr uint32_t IDESC_PV = (2u << 4) | (1u << 7) | (0u << 10) | (1u << 15) | ((64u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void mma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ uint32_t okey(float x) {       // order-preserving float -> uint
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float okey_inv(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k ^ 0x80000000u) : ~k);
}

struct Bars {
  uint64_t full[STAGES], empty[STAGES];
  uint64_t s_full, s_empty, p_ready, o_full, o_empty;
};

template <int G>
__global__ void __launch_bounds__(192, 2)
attn_decode_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                      const DecodeParamsV2 p) {
  pdl_wait();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* pb = smem + STAGES * STAGE_BYTES;               // 4 B tiles of P, 2 KB each
  uint8_t* qb = pb + 4 * PB_BYTES;                         // queries as a B tile, 2 KB
  Bars* bars = reinterpret_cast<Bars*>(qb + PB_BYTES);
  CtaAbort* ab = reinterpret_cast<CtaAbort*>(bars + 1);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ab + 1);

  __shared__ float sdq[8][4];
  __shared__ uint32_t s_red[2][4][12];
  __shared__ int s_ok[2][4];
  __shared__ int s_abort;
  __shared__ float s_l[4][8];
  __shared__ float sm_m[1][G], sm_l[1][G];
  __shared__ float sm_o[1][G][HD];
  __shared__ int s_last;
  __shared__ float red[4];

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
  const int tb0 = r0 & ~(PAGE - 1);
  const int ntiles = r1 > r0 ? (r1 - tb0 + TILE - 1) / TILE : 0;
  const long long n_pages = p.num_slots / PAGE;
  const int* bt = p.block_table + (long long)seq * p.max_blocks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    mbar_init(&bars->s_full, 1);
    mbar_init(&bars->s_empty, 4);
    mbar_init(&bars->p_ready, 4);
    mbar_init(&bars->o_full, 1);
    mbar_init(&bars->o_empty, 4);
    ab->flag = 0;
    fence_mbar_init();
  }
  // zero the B tiles (their unused rows must stay zero), then stage the queries as int8
  for (int i = threadIdx.x; i < 5 * PB_BYTES / 16; i += blockDim.x)
    reinterpret_cast<uint4*>(pb)[i] = make_uint4(0, 0, 0, 0);
  __syncthreads();
  if (warp < 4) {
    for (int g = warp; g < G; g += 4) {
      const __nv_bfloat16* qp = p.q + ((long long)row * p.n_q + kvh * G + g) * HD + lane * 4;
      float v[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) v[e] = bf2f(qp[e]);
      float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      const float d = amax * (1.f / 127.f);
      const float id = d > 0.f ? 1.f / d : 0.f;
      char4 c;
      c.x = (signed char)__float2int_rn(v[0] * id);
      c.y = (signed char)__float2int_rn(v[1] * id);
      c.z = (signed char)__float2int_rn(v[2] * id);
      c.w = (signed char)__float2int_rn(v[3] * id);
      // row g, bytes 4 lane .. 4 lane + 3 of a 128-byte-swizzled K-major tile
      *reinterpret_cast<char4*>(qb + sw128_offset(g, lane >> 2) + (lane & 3) * 4) = c;
      if ((lane & 7) == 0) sdq[g][lane >> 3] = d * p.scale_log2;
    }
  }
  if (warp == 5) tmem_alloc(tmem_slot, TMEM_COLS);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_s = tmem, tmem_o = tmem + 64;
  // only now may the next kernel be scheduled: it allocates tensor memory in its prologue, before it waits
  // for this one, and must not take the columns this CTA was about to ask for
  pdl_launch();

  if (warp == 4) {
    // ------------------------------ TMA producer ------------------------------
    if (elect_one()) {
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      for (int it = 0; it < ntiles; ++it) {
        const int st = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait(&bars->empty[st], ph ^ 1, ab, p.status, 31)) break;
        mbar_expect_tx(&bars->full[st], STAGE_BYTES);
        uint8_t* ks = smem + st * STAGE_BYTES;
        uint8_t* vs = ks + TILE * HD;
        const int pg0 = (tb0 + it * TILE) / PAGE;
#pragma unroll
        for (int j = 0; j < TILE / PAGE; ++j) {
          long long blk = 0;
          if (pg0 + j < p.max_blocks && (pg0 + j) * PAGE < r1) blk = bt[pg0 + j];
          if (blk < 0 || blk >= n_pages) {
            if (p.status) atomicCAS(p.status, 0, LK_ERR_BOUNDS | (6 << 8));
            blk = 0;
          }
          tma_load_3d(ks + j * PAGE * HD, &tmK, &bars->full[st], 0, kvh, (int)(blk * PAGE));
          tma_load_3d(vs + j * PAGE * HD, &tmV, &bars->full[st], 0, kvh, (int)(blk * PAGE));
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------ MMA issuer ------------------------------
    if (elect_one()) {
      const uint64_t qdesc = make_desc_sw128(smem_u32(qb));
      auto issue_qk = [&](int it) -> bool {
        const int st = it % STAGES;
        if (!mbar_wait(&bars->full[st], (it / STAGES) & 1, ab, p.status, 32)) return false;
        if (!mbar_wait(&bars->s_empty, (it & 1) ^ 1, ab, p.status, 33)) return false;
        tc_fence_after();
        const uint64_t kdesc = make_desc_sw128(smem_u32(smem + st * STAGE_BYTES));
#pragma unroll
        for (int b = 0; b < 4; ++b)          // block b: 32 bytes further along the 128-byte rows
          mma_i8(tmem_s + 16 * b, kdesc + (uint64_t)(2 * b), qdesc + (uint64_t)(2 * b), IDESC_QK, 0u);
        mma_commit(&bars->s_full);
        return true;
      };
      bool ok = ntiles > 0 && issue_qk(0);
      for (int it = 0; it < ntiles && ok; ++it) {
        const int st = it % STAGES;
        if (it + 1 < ntiles) ok = issue_qk(it + 1);       // the next tile's scores overlap this tile's softmax
        if (!ok) break;
        if (!mbar_wait(&bars->p_ready, it & 1, ab, p.status, 34)) break;
        if (!mbar_wait(&bars->o_empty, (it & 1) ^ 1, ab, p.status, 35)) break;
        tc_fence_after();
        const uint64_t vdesc = make_desc_sw128(smem_u32(smem + st * STAGE_BYTES + TILE * HD));
        // the four blocks' B tiles are stacked (64 rows): one N = 64 MMA per 32 keys puts block b's
        // sums into columns 16 b .. 16 b + 15
        const uint64_t pdesc = make_desc_sw128(smem_u32(pb));
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)       // 32 keys per step: 4 KB down the V tile, 32 bytes along P's rows
          mma_i8(tmem_o, vdesc + (uint64_t)(ks * 256), pdesc + (uint64_t)(2 * ks), IDESC_PV, ks > 0 ? 1u : 0u);
        mma_commit(&bars->o_full);
        mma_commit(&bars->empty[st]);         // K and V of this stage have been read by the tensor core
      }
    }
  } else {
    // ------------------------------ softmax / output threads ------------------------------
    const int t = threadIdx.x;                       // key of the tile, later dim of the output
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    float m_run[G], l_run[G], O[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      m_run[g] = -INFINITY;
      l_run[g] = 0.f;
      O[g] = 0.f;
    }
    float dq[G][4];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int b = 0; b < 4; ++b) dq[g][b] = sdq[g][b];
    auto key_slot = [&](int it) -> long long {
      const int pg = (tb0 + it * TILE) / PAGE + (t >> 4);
      long long blk = 0;
      if (it < ntiles && pg < p.max_blocks && pg * PAGE < r1) blk = bt[pg];
      if (blk < 0 || blk >= n_pages) blk = 0;
      return blk * PAGE + (t & 15);
    };
    // Scales are requested one tile ahead and page numbers two tiles ahead, so neither of the two
    // dependent global loads is waited for inside a tile.
    auto load_scales = [&](long long slot, uint2& kr, uint2& vr) {
      kr = *reinterpret_cast<const uint2*>(p.k_scale + (slot * p.n_kv + kvh) * 4);
      vr = *reinterpret_cast<const uint2*>(p.v_scale + (slot * p.n_kv + kvh) * 4);
    };
    uint2 kraw_n, vraw_n;
    load_scales(key_slot(0), kraw_n, vraw_n);
    long long slot_next = key_slot(1);
    bool ok = true;
    for (int it = 0; it < ntiles; ++it) {
      const uint2 kraw = kraw_n, vraw = vraw_n;
      load_scales(slot_next, kraw_n, vraw_n);            // tile it + 1 (slot 0 of page 0 past the end)
      slot_next = key_slot(it + 2);
      const int kpos = tb0 + it * TILE + t;
      const bool valid = kpos >= r0 && kpos < r1;
      float dk[4], dv[4];
      {
        const __half2 k01 = *reinterpret_cast<const __half2*>(&kraw.x), k23 = *reinterpret_cast<const __half2*>(&kraw.y);
        const __half2 v01 = *reinterpret_cast<const __half2*>(&vraw.x), v23 = *reinterpret_cast<const __half2*>(&vraw.y);
        dk[0] = __low2float(k01); dk[1] = __high2float(k01); dk[2] = __low2float(k23); dk[3] = __high2float(k23);
        dv[0] = __low2float(v01); dv[1] = __high2float(v01); dv[2] = __low2float(v23); dv[3] = __high2float(v23);
        if (!valid) dv[0] = dv[1] = dv[2] = dv[3] = 0.f;
      }
      // A failed (timed-out) wait never leaves the loop on its own: every thread still meets the
      // others at this tile's barrier, where the four warps agree on whether to go on.
      if (ok) ok = mbar_wait(&bars->s_full, it & 1, ab, p.status, 36);
      float s[G];
#pragma unroll
      for (int g = 0; g < G; ++g) s[g] = 0.f;
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          uint32_t r[8];
          tmem_ld8(tmem_s + lane_addr + 16 * b, r);
          tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < G; ++g) s[g] = fmaf((float)(int)r[g], dk[b] * dq[g][b], s[g]);
        }
        tc_fence_before();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->s_empty);       // the next tile's scores may overwrite S
      // tile maxima: scores per head, value scales per block
      uint32_t* rw = s_red[it & 1][warp];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const uint32_t k = __reduce_max_sync(0xffffffffu, okey(valid ? s[g] : -INFINITY));
        if (lane == 0) rw[g] = k;
      }
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const uint32_t k = __reduce_max_sync(0xffffffffu, __float_as_uint(dv[b]));
        if (lane == 0) rw[8 + b] = k;
      }
      {
        const int warp_ok = __all_sync(0xffffffffu, ok);
        if (lane == 0) s_ok[it & 1][warp] = warp_ok;
      }
      asm volatile("bar.sync 3, 128;" ::: "memory");
      ok = s_ok[it & 1][0] && s_ok[it & 1][1] && s_ok[it & 1][2] && s_ok[it & 1][3];
      if (!ok) break;                                   // the same decision in all 128 threads
      float alpha[G], pr[G], sfac[4], qinv[4];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const uint32_t k = max(max(s_red[it & 1][0][g], s_red[it & 1][1][g]),
                               max(s_red[it & 1][2][g], s_red[it & 1][3][g]));
        const float mt = okey_inv(k);
        const float mn = fmaxf(m_run[g], mt);
        alpha[g] = (mn > -INFINITY) ? exp2f(m_run[g] - mn) : 1.f;
        pr[g] = (valid && mn > -INFINITY) ? exp2f(s[g] - mn) : 0.f;
        l_run[g] = l_run[g] * alpha[g] + pr[g];
        m_run[g] = mn;
      }
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const uint32_t k = max(max(s_red[it & 1][0][8 + b], s_red[it & 1][1][8 + b]),
                               max(s_red[it & 1][2][8 + b], s_red[it & 1][3][8 + b]));
        const float dmax = __uint_as_float(k);
        sfac[b] = dmax * (1.f / 32767.f);
        qinv[b] = dmax > 0.f ? 32767.f / dmax : 0.f;
      }
      // P_b[t, g] as two bytes: high byte in row g, low byte in row 8 + g, column t
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const float f = dv[b] * qinv[b];
        uint8_t* tile = pb + b * PB_BYTES;
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const uint32_t q = min(__float2uint_rn(pr[g] * f), 32767u);
          tile[sw128_offset(g, t >> 4) + (t & 15)] = (uint8_t)(q >> 8);
          tile[sw128_offset(8 + g, t >> 4) + (t & 15)] = (uint8_t)(q & 255u);
        }
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_ready);
      // this tile's P.V: thread t is now output dim t, block t / 32 = its warp
      ok = mbar_wait(&bars->o_full, it & 1, ab, p.status, 37);
      if (ok) {
        tc_fence_after();
        uint32_t r[16];
        tmem_ld16(tmem_o + lane_addr + 16 * warp, r);
        tmem_ld_wait();
        const float sf = sfac[warp];
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float val = (float)(int)r[g] * 256.f + (float)(int)r[8 + g];
          O[g] = fmaf(val, sf, O[g] * alpha[g]);
        }
        tc_fence_before();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->o_empty);
    }
    // the row sums are per thread (per key): add them up over the 128 threads
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float ws = warp_sum(l_run[g]);
      if (lane == 0) s_l[warp][g] = ws;
    }
    asm volatile("bar.sync 2, 128;" ::: "memory");
#pragma unroll
    for (int g = 0; g < G; ++g) {
      if (t == 0) {
        sm_m[0][g] = m_run[g];
        sm_l[0][g] = s_l[0][g] + s_l[1][g] + s_l[2][g] + s_l[3][g];
      }
      sm_o[0][g][t] = O[g];
    }
    if (t == 0) s_abort = ab->flag;                     // one reading, so all 128 threads agree
    asm volatile("bar.sync 2, 128;" ::: "memory");
    if (!s_abort) decode_finish<HD, G, 1>(p, row, kvh, split, nsplit, sm_m, sm_l, sm_o, &s_last, red, t);
  }
  // TMEM goes back only when nobody can still be reading it
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

int make_cache_tmap(CUtensorMap* tm, const void* base, long long num_slots, int n_kv) {
  PFN_cuTensorMapEncodeTiled enc = lkh::get_encode_fn();
  if (!enc) return LKH_NO_DRIVER;
  if (reinterpret_cast<uintptr_t>(base) & 15) return LKH_BAD_ARG;
  cuuint64_t gdim[3] = {(cuuint64_t)HD, (cuuint64_t)n_kv, (cuuint64_t)num_slots};
  cuuint64_t gstr[2] = {(cuuint64_t)HD, (cuuint64_t)n_kv * HD};
  cuuint32_t box[3] = {HD, 1, PAGE};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), gdim, gstr, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? LKH_OK : LKH_TMAP_FAIL;
}

template <int G>
int launch(const CUtensorMap& tmK, const CUtensorMap& tmV, const DecodeParamsV2& p, dim3 grid, cudaStream_t st) {
  constexpr int SMEM = STAGES * STAGE_BYTES + 5 * PB_BYTES + 256 + 1024;
  auto kern = attn_decode_tc_kernel<G>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  lkh::launch_pdl(kern, grid, dim3(192), SMEM, st, tmK, tmV, p);
  lkh::count_launch();
  return lkh::launch_status();
}

}  // namespace

// Same arguments as lk_attn_decode; serves head_dim 128, q8 cache, 16-token pages, group <= 8.
LK_API int lk_attn_decode_tc(const LkDecodeArgs* a, void* stream) {
  if (a->rows <= 0) return LKH_OK;
  if (a->hd != HD || !a->kv_q8 || a->block_size != PAGE || a->n_kv <= 0 || a->n_q % a->n_kv) return LKH_BAD_ARG;
  const int G = a->n_q / a->n_kv;
  const int nsplit = a->nsplit < 1 ? 1 : a->nsplit;
  if (nsplit > 1) {
    if (!a->ws || !a->counters) return LKH_BAD_ARG;
    if (lk_attn_decode_ws_floats(a->rows, a->n_q, a->n_kv, a->hd, nsplit) > a->ws_floats ||
        (long long)a->rows * a->n_kv > a->n_counters)
      return LKH_TOO_LARGE;
  }
  if (a->out_fp8 && !a->out_scales_t) return LKH_BAD_ARG;
  CUtensorMap tmK, tmV;
  int rc = make_cache_tmap(&tmK, a->k_cache, a->num_slots, a->n_kv);
  if (rc != LKH_OK) return rc;
  rc = make_cache_tmap(&tmV, a->v_cache, a->num_slots, a->n_kv);
  if (rc != LKH_OK) return rc;
  DecodeParamsV2 p;
  p.q = (const __nv_bfloat16*)a->q;
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
  dim3 grid(a->n_kv, a->rows, nsplit);
  cudaStream_t st = (cudaStream_t)stream;
  switch (G) {
    case 1: return launch<1>(tmK, tmV, p, grid, st);
    case 2: return launch<2>(tmK, tmV, p, grid, st);
    case 4: return launch<4>(tmK, tmV, p, grid, st);
    case 8: return launch<8>(tmK, tmV, p, grid, st);
    default: return LKH_BAD_ARG;
  }
}
