// Flash prefill attention on tcgen05 for GQA: causal, optional sliding window, optional
// attention sinks, variable-length batches, query rows that start at any position of their
// sequence (chunked prefill, prompts with a cached prefix, speculative verify windows).
//
// One CTA = 128 score rows = (128 / G) consecutive query tokens x the G query heads that share
// one kv head, so every K / V tile is loaded once for the whole group.  The TMA box
// {64 dims, G heads, 128/G tokens} lands the rows token-major in shared memory, which is the
// row order the MMA wants.  Keys arrive as dense bf16 [tok, n_kv, hd] and values transposed
// [n_kv, hd, tok] (lk_kv_gather writes both from the paged cache), so all four MMA operands
// are K-major with the 128-byte swizzle.
//
// Per 128-key tile:  S = Q K^T (tcgen05, fp32 in TMEM columns 0..127)
//                    softmax warps: one row per thread, two passes over TMEM (max, then
//                      exp2 + row sum), P written as bf16 into swizzled shared memory
//                    O_tile = P V (tcgen05, TMEM columns 128..128+hd), folded into fp32
//                      registers with the usual running-max rescale.
// Warp 4 issues the MMAs, warp 5 the TMA loads (two K/V stages), warps 0-3 do softmax.
//
// Counterpart in the reference: cuda/flash_prefill_gqa.cu (mma.sync m16n8k16, cp.async).
#include "common.cuh"
#include "host_common.h"
#include "loken_cuda.h"
#include "tc100.cuh"

using namespace lk;

namespace {

struct PrefillParams {
  __nv_bfloat16* out;
  const float* sinks;
  const int* tile_seq;
  const int* tile_q0;
  const int* q_start;
  const int* q_len;
  const int* kv_off;
  const int* kv_len;
  int* status;
  int n_q, n_kv, window;
  int g_real;          // query heads per kv head in the model; the tile holds G >= g_real head slots (a power of two)
  float scale_log2;
};

template <int HD>
struct PrefillSmem {
  static constexpr int Q_BYTES = 128 * HD * 2;          // HD/64 atoms of [128 rows x 128 B]
  static constexpr int K_BYTES = 128 * HD * 2;          // per stage
  static constexpr int V_BYTES = HD * 128 * 2;          // per stage: 2 atoms of [HD rows x 128 B]
  static constexpr int P_BYTES = 128 * 128 * 2;         // 2 atoms of [128 rows x 128 B]
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + Q_BYTES;
  static constexpr int V_OFF = K_OFF + 2 * K_BYTES;
  static constexpr int P_OFF = V_OFF + 2 * V_BYTES;
  static constexpr int BAR_OFF = P_OFF + P_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

template <int HD, int G>
__global__ void __launch_bounds__(192, 1)
attn_prefill_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const PrefillParams p) {
  using S = PrefillSmem<HD>;
  constexpr int TQ = 128 / G;
  constexpr int NQA = HD / 64;  // 128-byte atoms along the head dimension
  constexpr uint32_t TMEM_COLS = 256;
  constexpr float LOG2E = 1.4426950408889634f;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::BAR_OFF);
  uint64_t* q_full = bars + 0;
  uint64_t* kv_full = bars + 1;    // [2]
  uint64_t* kv_empty = bars + 3;   // [2]
  uint64_t* s_full = bars + 5;
  uint64_t* p_ready = bars + 6;
  uint64_t* o_full = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  CtaAbort* ab = reinterpret_cast<CtaAbort*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, kvh = blockIdx.y;
  const int seq = p.tile_seq[tile];
  const int tq0 = p.tile_q0[tile];
  const int qlen = p.q_len[seq], kvlen = p.kv_len[seq];
  const int qrow0 = p.q_start[seq] + tq0;
  const int kvoff = p.kv_off[seq];
  const int pos0 = kvlen - qlen;  // position of the sequence's first query token
  const int first_pos = pos0 + tq0;
  const int last_pos = pos0 + min(tq0 + TQ, qlen) - 1;
  const int kt_begin = (p.window > 0) ? max(0, first_pos - p.window + 1) / 128 : 0;
  const int kt_end = last_pos / 128;  // inclusive
  const int ntiles = max(0, kt_end - kt_begin + 1);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_ready, 128);
    mbar_init(o_full, 1);
    ab->flag = 0;
    fence_mbar_init();
  }
  if (warp == 4) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 5) {
    // ------------------------------ TMA producer ------------------------------
    if (elect_one()) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, S::Q_BYTES);
#pragma unroll
      for (int a = 0; a < NQA; ++a)
        // G head slots from the group's first head on: slots past g_real hold the next group's heads (zeros
        // past the last head) and are never stored
        tma_load_3d(smem + S::Q_OFF + a * 16384, &tmQ, q_full, a * 64, kvh * p.g_real, qrow0);
      for (int it = 0; it < ntiles; ++it) {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(&kv_empty[st], ph ^ 1, ab, p.status, 11)) break;
        mbar_expect_tx(&kv_full[st], S::K_BYTES + S::V_BYTES);
        const int key0 = kvoff + (kt_begin + it) * 128;
#pragma unroll
        for (int a = 0; a < NQA; ++a)
          tma_load_3d(smem + S::K_OFF + st * S::K_BYTES + a * 16384, &tmK, &kv_full[st], a * 64, kvh, key0);
#pragma unroll
        for (int a = 0; a < 2; ++a)
          tma_load_3d(smem + S::V_OFF + st * S::V_BYTES + a * (HD * 128), &tmV, &kv_full[st], key0 + a * 64, 0,
                      kvh);
      }
    }
  } else if (warp == 4) {
    // ------------------------------ MMA issuer --------------------------------
    if (elect_one()) {
      constexpr uint32_t idesc_qk = make_idesc(1, 1, 128, 128);
      constexpr uint32_t idesc_pv = make_idesc(1, 1, 128, HD);
      bool ok = mbar_wait(q_full, 0, ab, p.status, 12);
      for (int it = 0; it < ntiles && ok; ++it) {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        ok = mbar_wait(&kv_full[st], ph, ab, p.status, 13);
        if (!ok) break;
        tc_fence_after();
        const uint32_t qa = smem_u32(smem + S::Q_OFF);
        const uint32_t ka = smem_u32(smem + S::K_OFF + st * S::K_BYTES);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint64_t ad = make_desc_sw128(qa + (k >> 2) * 16384) + 2 * (k & 3);
          const uint64_t bd = make_desc_sw128(ka + (k >> 2) * 16384) + 2 * (k & 3);
          mma_bf16(tmem_base, ad, bd, idesc_qk, k > 0 ? 1u : 0u);
        }
        mma_commit(s_full);
        ok = mbar_wait(p_ready, it & 1, ab, p.status, 14);
        if (!ok) break;
        tc_fence_after();
        const uint32_t pa = smem_u32(smem + S::P_OFF);
        const uint32_t va = smem_u32(smem + S::V_OFF + st * S::V_BYTES);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint64_t ad = make_desc_sw128(pa + (k >> 2) * 16384) + 2 * (k & 3);
          const uint64_t bd = make_desc_sw128(va + (k >> 2) * (HD * 128)) + 2 * (k & 3);
          mma_bf16(tmem_base + 128, ad, bd, idesc_pv, k > 0 ? 1u : 0u);
        }
        mma_commit(o_full);
        mma_commit(&kv_empty[st]);
      }
    }
  } else {
    // ------------------------------ softmax + output ----------------------------
    const int r = threadIdx.x;              // score row = TMEM lane
    const int tq = r / G, g = r % G;
    const int qi = tq0 + tq;
    const bool row_ok = qi < qlen && g < p.g_real;
    const int pos = pos0 + qi;
    const int lo = (p.window > 0) ? max(0, pos - p.window + 1) : 0;
    const int head = kvh * p.g_real + g;
    const uint32_t tw = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    uint8_t* psm = smem + S::P_OFF;

    float m = -INFINITY, l = 0.f;
    if (p.sinks && row_ok) {
      m = p.sinks[head] * LOG2E;
      l = 1.f;
    }
    float O[HD];
#pragma unroll
    for (int d = 0; d < HD; ++d) O[d] = 0.f;

    bool ok = true;
    for (int it = 0; it < ntiles && ok; ++it) {
      const int j0 = (kt_begin + it) * 128;
      ok = mbar_wait(s_full, it & 1, ab, p.status, 15);
      if (!ok) break;
      tc_fence_after();
      // pass 1: row maximum of the admissible scores
      float tmax = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t sv[32];
        tmem_ld32(tw + c * 32, sv);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const int j = j0 + c * 32 + e;
          if (row_ok && j >= lo && j <= pos) tmax = fmaxf(tmax, __uint_as_float(sv[e]) * p.scale_log2);
        }
      }
      const float mn = fmaxf(m, tmax);
      const float alpha = (mn > -INFINITY) ? exp2f(m - mn) : 1.f;
      // pass 2: probabilities -> bf16 P tile in swizzled shared memory
      float psum = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t sv[32];
        tmem_ld32(tw + c * 32, sv);
        tmem_ld_wait();
        float pv[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const int j = j0 + c * 32 + e;
          const bool keep = row_ok && j >= lo && j <= pos;
          pv[e] = keep ? exp2f(__uint_as_float(sv[e]) * p.scale_log2 - mn) : 0.f;
          psum += pv[e];
        }
#pragma unroll
        for (int q8 = 0; q8 < 4; ++q8) {
          uint4 pk;
          __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
          for (int e = 0; e < 4; ++e) h2[e] = __floats2bfloat162_rn(pv[q8 * 8 + 2 * e], pv[q8 * 8 + 2 * e + 1]);
          const int col = c * 32 + q8 * 8;           // key column inside the tile
          const uint32_t off = (col >> 6) * 16384u + sw128_offset(r, (col & 63) >> 3);
          *reinterpret_cast<uint4*>(psm + off) = pk;
        }
      }
      l = l * alpha + psum;
      m = mn;
      // fold the previous tile's P V product before this tile's rescale
      if (it > 0) {
        ok = mbar_wait(o_full, (it - 1) & 1, ab, p.status, 16);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t ov[32];
          tmem_ld32(tw + 128 + c * 32, ov);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) O[c * 32 + e] = (O[c * 32 + e] + __uint_as_float(ov[e])) * alpha;
        }
      }
      tc_fence_before();
      fence_async_smem();
      mbar_arrive(p_ready);
    }
    if (ok && ntiles > 0) {
      ok = mbar_wait(o_full, (ntiles - 1) & 1, ab, p.status, 17);
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t ov[32];
          tmem_ld32(tw + 128 + c * 32, ov);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) O[c * 32 + e] += __uint_as_float(ov[e]);
        }
        tc_fence_before();
      }
    }
    if (ok && row_ok) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = p.out + (long long)(qrow0 + tq) * p.n_q * HD + head * HD;
#pragma unroll
      for (int d = 0; d < HD; d += 8) {
        uint4 pk;
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
        for (int e = 0; e < 4; ++e) h2[e] = __floats2bfloat162_rn(O[d + 2 * e] * inv, O[d + 2 * e + 1] * inv);
        *reinterpret_cast<uint4*>(dst + d) = pk;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    if (ab->flag) {
      for (int t = 0; t < 64; ++t) __nanosleep(2000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

inline int make_tmap_3d_box(CUtensorMap* tm, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t ld1,
                            uint64_t ld2, uint32_t b0, uint32_t b1, uint32_t b2) {
  PFN_cuTensorMapEncodeTiled enc = lkh::get_encode_fn();
  if (!enc) return LKH_NO_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld1 & 15) || (ld2 & 15) || b0 * 2 != 128 || b1 > 256 || b2 > 256)
    return LKH_BAD_ARG;
  cuuint64_t gdim[3] = {d0, d1, d2};
  cuuint64_t gstr[2] = {ld1, ld2};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), gdim, gstr, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? LKH_OK : LKH_TMAP_FAIL;
}

template <int HD, int G>
int launch(const LkPrefillArgs& a, const PrefillParams& p, cudaStream_t st) {
  using S = PrefillSmem<HD>;
  CUtensorMap tmQ, tmK, tmV;
  int rc = make_tmap_3d_box(&tmQ, a.q, HD, a.n_q, a.total_q, (uint64_t)HD * 2, (uint64_t)a.n_q * HD * 2, 64, G,
                            128 / G);
  if (rc) return rc;
  rc = make_tmap_3d_box(&tmK, a.k, HD, a.n_kv, a.total_kv_pad, (uint64_t)HD * 2, (uint64_t)a.n_kv * HD * 2, 64, 1,
                        128);
  if (rc) return rc;
  rc = make_tmap_3d_box(&tmV, a.vt, a.total_kv_pad, HD, a.n_kv, (uint64_t)a.total_kv_pad * 2,
                        (uint64_t)a.total_kv_pad * HD * 2, 64, HD, 1);
  if (rc) return rc;
  auto kern = attn_prefill_kernel<HD, G>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  dim3 grid(a.n_tiles, a.n_kv);
  kern<<<grid, 192, S::TOTAL, st>>>(tmQ, tmK, tmV, p);
  lkh::count_launch();
  return lkh::launch_status();
}

}  // namespace

LK_API int lk_attn_prefill(const LkPrefillArgs* args, void* stream) {
  const LkPrefillArgs& a = *args;
  if (a.n_tiles <= 0) return LKH_OK;
  if (a.n_kv <= 0 || a.n_q % a.n_kv || (a.total_kv_pad % 128)) return LKH_BAD_ARG;
  // group sizes that are not a power of two (3, 5, 6, 7: Llama-3.2-3B, Qwen2.5-14B / 32B) run in the next
  // larger tile shape with the spare head slots idle
  const int g_real = a.n_q / a.n_kv;
  const int G = g_real <= 1 ? 1 : g_real <= 2 ? 2 : g_real <= 4 ? 4 : 8;
  if (g_real > 8) return LKH_BAD_ARG;
  PrefillParams p;
  p.g_real = g_real;
  p.out = (__nv_bfloat16*)a.out;
  p.sinks = a.sinks;
  p.tile_seq = a.tile_seq; p.tile_q0 = a.tile_q0;
  p.q_start = a.q_start; p.q_len = a.q_len; p.kv_off = a.kv_off; p.kv_len = a.kv_len;
  p.status = a.status;
  p.n_q = a.n_q; p.n_kv = a.n_kv; p.window = a.window;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  cudaStream_t st = (cudaStream_t)stream;
#define LK_PF(HD, GG) \
  if (a.hd == HD && G == GG) return launch<HD, GG>(a, p, st)
  LK_PF(128, 1); LK_PF(128, 2); LK_PF(128, 4); LK_PF(128, 8);
  LK_PF(64, 1); LK_PF(64, 2); LK_PF(64, 4); LK_PF(64, 8);
#undef LK_PF
  return LKH_BAD_ARG;
}
