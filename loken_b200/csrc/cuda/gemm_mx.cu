// Block-scaled (microscaling) GEMM on the 5th-generation tensor cores:
//
//     C[i, j] = sum_k  A[i, k] * 2^(SFA[i, k/32] - 127)  *  B[j, k] * 2^(SFB[j, k/32] - 127)
//
//   A: MXFP4 weights as the file stores them: E2M1 nibbles [Ra, K/2] (value k of a row in byte k/2,
//      low nibble for even k) and one E8M0 exponent per 32 values [Ra, sfa_ld]; rows ride the MMA M side
//   B: token rows quantised to e4m3 with one E8M0 exponent per 32 values (mx_quant.cu); rows ride N
//
// The scales are applied by the hardware: `tcgen05.mma.kind::mxf8f6f4.block_scale` takes one
// exponent per operand row per 32 values of K from tensor memory, so nothing is dequantised and the
// accumulator runs over all of K in TMEM.  Per stage (128 values of K):
//   * warp 0 (one lane) brings the token tile by TMA (e4m3, 128-byte swizzle, as the fp8 GEMM does) and
//     the weight tile's packed nibbles (128 rows x 64 bytes, unswizzled) into a staging buffer;
//   * eight copy warps re-lay the staged nibbles as the tensor core's 4-bit-in-8-bit container layout
//     (16 values = 8 bytes of nibbles followed by 8 bytes of padding in every 16-byte chunk) in the
//     swizzled K-major tile: one 16-byte shared load and two 16-byte shared stores per 32 values, no
//     arithmetic on the values, nothing of the weight stream waits in registers; and they lay the
//     stage's exponents (fetched sixteen stages ahead) out as the 32 x 16-byte block `tcgen05.cp`
//     copies (row r of the tile in lane r % 32, column r / 32, one byte per 32 values of K);
//   * warp 1 (one lane) copies both exponent blocks to tensor memory with `tcgen05.cp.32x128b.warpx4`
//     (four column sets in rotation, so a copy never waits for the MMAs that still read the last one)
//     and issues four K = 32 MMAs, selecting the exponent byte through the instruction descriptor;
//   * four epilogue warps read the finished tile with `tcgen05.ld` and store it (bias, strides and
//     bounds as in gemm_tc.cuh).
// Persistent over output tiles; grouped (mixture of experts) launches walk the same device-side
// tile list as the bf16 grouped GEMM.  Every wait is bounded and reports through the status word.
//
// The same kernel runs block-scaled fp8 checkpoints whose scales are powers of two (E8M0, the
// `.scale` variant of 128x128-block fp8 files) [AKIND = 1]: e4m3 weight tiles arrive by TMA, the
// block's exponent is replicated over its 128 rows and four K sub-blocks, and the activations'
// per-token-per-128 scales (powers of two by construction, elementwise.cu) give the token exponents.
// That replaces the per-K-block fold through registers of gemm_tc_kernel<KIND_F8BLK> with one
// accumulation over all of K in tensor memory.  Dense launches split K over the CTAs when the tile
// count does not fill the chip: partials go to a workspace and the last-arriving split sums them in
// split order (deterministic), as in gemm_tc.cuh.
//
// The reference decodes MXFP4 with a pre-doubled int8 table and dp4a against q8 activations
// (cuda/moe/mxfp4_moe.cuh:14-40, cuda/moe/moe_gguf.cu:405-1340); its bar for 8-bit activations is
// 2e-2 of the largest expected output (src/inference/generic_transformer/moe_weights.rs:2977-2984).
#include "gemm_tc.cuh"
#include "host_common.h"
#include "loken_cuda.h"
#include <string.h>

using namespace lk;

namespace {

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

constexpr int MX_COPY_WARPS = 8;
constexpr int MX_THREADS = 64 + 128 + 32 * MX_COPY_WARPS;   // TMA, MMA, 4 epilogue, 8 copy warps

// idesc of kind::mxf8f6f4.block_scale: a = E2M1 (5), b = E4M3 (0), E8M0 scales, both K-major
__host__ __device__ constexpr uint32_t make_idesc_mx(uint32_t a_fmt, uint32_t b_fmt, uint32_t M, uint32_t N) {
  return (a_fmt << 7) | (b_fmt << 10) | ((N >> 3) << 17) | (1u << 23) | ((M >> 4) << 24);
}
// no-swizzle K-major descriptor of a 32-row x 16-byte block whose 8-row groups are 128 bytes apart
__device__ __forceinline__ uint64_t make_desc_sf(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(128 >> 4) << 32;     // stride byte offset between 8-row groups
  d |= static_cast<uint64_t>(1) << 46;            // descriptor version
  return d;
}
__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void mma_mx(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                       uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
      : "memory");
}

// MT = weight tiles (of 128 rows) that share one token tile per stage
// the strided scalar store of gemm_tc.cuh, kept out of line: it is the rare path (fp32 or odd-pitch outputs)
template <int CH>
__device__ __noinline__ void store_chunk_slow(const GemmParams& p, const TileCtx& t, int i, int j0, const float (&v)[CH]) {
  store_chunk<CH>(p, t, i, j0, v);
}

template <int BN, int STAGES, int AKIND, int MT>
struct MxSmem {
  static constexpr int A_TILE = 128 * 128;
  static constexpr int A_BYTES = MT * A_TILE;
  static constexpr int B_BYTES = BN * 128;
  static constexpr int SF_BYTES = ((MT + 1) * 512 + 1023) / 1024 * 1024;   // exponents of one stage: MT A blocks + B block
  static constexpr int RAW_BYTES = AKIND == 0 ? 128 * 64 : 0;       // staged nibbles of the weight tile
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SF_BYTES + RAW_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int EPI_OFFSET = BAR_OFFSET + 512;
  static constexpr int EPI_BYTES = 2 * (BN >= 32 ? 32 : 16) * 128 * 2;   // two chunks of [token][128 features] bf16
  static constexpr int TOTAL = EPI_OFFSET + EPI_BYTES + 1024;
};
constexpr int MX_SF_SETS = 4;      // exponent column sets in tensor memory (4 columns per operand tile each)

// AKIND 0: MXFP4 weights moved by the copy warps; 1: e4m3 weights by TMA with 128x128-block exponents.
// MT > 1 (dense e4m3 only): a unit of work is MT consecutive weight tiles against one token tile, so the
// token tile, which every weight tile re-reads through L2, is fetched once per MT * 16 KB of weights; the
// unit has MT accumulators side by side in tensor memory.
template <int BN, int STAGES, int AKIND, int MT>
__global__ void __launch_bounds__(MX_THREADS, 1)
gemm_mx_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ GemmParams p) {
  using S = MxSmem<BN, STAGES, AKIND, MT>;
  constexpr int CH = BN >= 32 ? 32 : 16;
  constexpr int NCH = BN / CH;
  constexpr uint32_t SF_COLS = 4 * MT + 4;               // a set: 4 columns of exponents per weight tile + 4 of the tokens
  constexpr int NACC = (2 * MT * BN + MX_SF_SETS * SF_COLS <= 512) ? 2 : 1;
  constexpr uint32_t ACC_COLS = MT * BN;
  constexpr uint32_t D_COLS = NACC * ACC_COLS;
  constexpr uint32_t NEED = D_COLS + SF_COLS * MX_SF_SETS;
  constexpr int AHEAD = MT == 1 ? 16 : MT == 2 ? 8 : 6;  // stages the exponent words are fetched ahead of their use
  static_assert(AKIND == 1 || MT == 1, "tile groups are built for the e4m3 form only");
  static_assert(NEED <= 512, "tensor memory");
  constexpr uint32_t TMEM_COLS = NEED <= 32 ? 32 : NEED <= 64 ? 64 : NEED <= 128 ? 128 : NEED <= 256 ? 256 : 512;
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 128, "BN");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* accf_bar = empty_bar + STAGES;
  uint64_t* acce_bar = accf_bar + NACC;
  uint64_t* raw_bar = acce_bar + NACC;       // staged nibbles of a stage have landed [STAGES]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(raw_bar + STAGES);
  CtaAbort* ab = reinterpret_cast<CtaAbort*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nkb_total = (p.K + 127) / 128;
  const bool grouped = p.g_rows_per_expert > 0;
  if (grouped) pdl_wait();
  // the first n_full tiles (a multiple of the grid) run whole; the remainder, which would be a nearly
  // empty last wave, is cut along K into `splits` units each and spread over all the CTAs
  const int splits = grouped ? 1 : p.splits;
  const int all_tiles = grouped ? (*p.g_ntiles) * p.tiles_a : p.tiles_a * p.tiles_b;
  // dense: p.n_full units of MT tiles each, then p.nrem units of p.rem_mt tiles each (every weight tile
  // belongs to exactly one unit; MT, rem_mt > 1 only with a single token tile)
  const int n_full = grouped ? all_tiles : p.n_full;
  const int nrem = grouped ? 0 : p.nrem;
  const int ntiles = n_full + nrem * splits;         // work units
  int* s_last = reinterpret_cast<int*>(tmem_slot + 2);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1 + MX_COPY_WARPS);
      mbar_init(&empty_bar[s], 1);
      mbar_init(&raw_bar[s], 1);
    }
    for (int s = 0; s < NACC; ++s) {
      mbar_init(&accf_bar[s], 1);
      mbar_init(&acce_bar[s], 4);
    }
    ab->flag = 0;
    *s_last = 0;
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();
  pdl_launch();
  if (p.prof && threadIdx.x == 0) p.prof[blockIdx.x * 8 + 4] = (long long)globaltimer_ns();

#define MX_TILE(u)                                                              \
  const bool whole_ = (u) < n_full;                                             \
  const int nsp = whole_ ? 1 : splits;                                          \
  const int split_ = whole_ ? 0 : ((u) - n_full) % splits;                      \
  const int tile_ = whole_ ? (u) : n_full + ((u) - n_full) / splits;            \
  const int kb_per = (nkb_total + nsp - 1) / nsp;                               \
  const int gi_ = grouped ? tile_ % p.tiles_a : tile_ / p.tiles_b;              \
  const int gfull_ = grouped ? 0 : n_full / p.tiles_b;                          \
  const int tile_a = (grouped || whole_) ? gi_ * MT : gfull_ * MT + (gi_ - gfull_) * p.rem_mt; \
  const int mt_here = MT == 1 ? 1 : max(1, min(whole_ ? MT : p.rem_mt, p.tiles_a - tile_a)); \
  const int tile_b = grouped ? tile_ / p.tiles_a : tile_ % p.tiles_b;           \
  const int kb_begin = split_ * kb_per;                                         \
  const int nkb = max(0, min(nkb_total, kb_begin + kb_per) - kb_begin);         \
  TileCtx tc;                                                                   \
  int b_row0;                                                                   \
  if (grouped) {                                                                \
    tc.a_base = p.g_tile_expert[tile_b] * p.g_rows_per_expert;                  \
    tc.ra_end = tc.a_base + p.g_rows_per_expert;                                \
    b_row0 = p.g_tile_row0[tile_b];                                             \
    tc.rb_end = b_row0 + p.g_tile_rows[tile_b];                                 \
  } else {                                                                      \
    tc.a_base = 0;                                                              \
    tc.ra_end = p.Ra;                                                           \
    b_row0 = tile_b * BN;                                                       \
    tc.rb_end = p.Rb;                                                           \
  }                                                                             \
  const int a_row0 = tc.a_base + tile_a * 128;

  if (warp == 0) {
    // ------------------------------ TMA producer: token tiles ------------------------------
    if (elect_one()) {
      tma_prefetch_desc(&tmB);
      tma_prefetch_desc(&tmA);
      int pit = 0;
      bool ok = true;
      long long w_empty = 0;
      for (int u = blockIdx.x; u < ntiles && ok; u += gridDim.x) {
        MX_TILE(u)
        (void)tile_a; (void)mt_here;
        for (int it = 0; it < nkb; ++it, ++pit) {
          const int s = pit % STAGES;
          const long long t0 = p.prof ? clock64() : 0;
          if (!mbar_wait(&empty_bar[s], ((pit / STAGES) & 1) ^ 1, ab, p.status, 1)) { ok = false; break; }
          if (p.prof) w_empty += clock64() - t0;
          uint8_t* sa = smem + s * S::STAGE_BYTES;
          if (AKIND == 1) {
            mbar_expect_tx(&full_bar[s], mt_here * S::A_TILE + S::B_BYTES);
#pragma unroll
            for (int m = 0; m < MT; ++m)
              if (m < mt_here) {
                // tile-major weights: tile (row block, K block) is 16 KB in one piece, 128 rows of 128 bytes
                if (p.a_tiled)
                  tma_load_2d(sa + m * S::A_TILE, &tmA, &full_bar[s], 0,
                              (((a_row0 >> 7) + m) * nkb_total + kb_begin + it) * 128);
                else
                  tma_load_2d(sa + m * S::A_TILE, &tmA, &full_bar[s], (kb_begin + it) * 128, a_row0 + m * 128);
              }
          } else {
            mbar_expect_tx(&full_bar[s], S::B_BYTES);
            mbar_expect_tx(&raw_bar[s], S::RAW_BYTES);
            tma_load_2d(sa + S::A_BYTES + S::B_BYTES + S::SF_BYTES, &tmA, &raw_bar[s], (kb_begin + it) * 64, a_row0);
          }
          tma_load_2d(sa + S::A_BYTES, &tmB, &full_bar[s], (kb_begin + it) * 128, b_row0);
        }
      }
      if (p.prof) p.prof[blockIdx.x * 8 + 0] = w_empty;
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_mx(AKIND == 0 ? 5 : 0, 0, 128, BN);
      const uint32_t sf_t0 = tmem_base + D_COLS;
      int mit = 0, ait = 0;
      bool ok = true;
      long long w_full = 0, w_acc = 0;
      const long long t_begin = p.prof ? clock64() : 0;
      for (int u = blockIdx.x; u < ntiles && ok; u += gridDim.x) {
        MX_TILE(u)
        (void)tile_a; (void)tile_b; (void)a_row0; (void)b_row0; (void)tc;
        if (nkb == 0) continue;
        const int buf = ait % NACC;
        const long long ta = p.prof ? clock64() : 0;
        if (!mbar_wait(&acce_bar[buf], ((ait / NACC) & 1) ^ 1, ab, p.status, 2)) { ok = false; break; }
        if (p.prof) w_acc += clock64() - ta;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * ACC_COLS;
        for (int it = 0; it < nkb; ++it, ++mit) {
          const int s = mit % STAGES;
          const long long t0 = p.prof ? clock64() : 0;
          if (!mbar_wait(&full_bar[s], (mit / STAGES) & 1, ab, p.status, 3)) { ok = false; break; }
          if (p.prof) w_full += clock64() - t0;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * S::STAGE_BYTES);
          const uint64_t bdesc = make_desc_sw128(a_addr + S::A_BYTES);
          const uint32_t sf_addr = a_addr + S::A_BYTES + S::B_BYTES;
          const uint32_t sfa_t = sf_t0 + (mit % MX_SF_SETS) * SF_COLS, sfb_t = sfa_t + 4 * MT;
          tmem_cp_sf(sfb_t, make_desc_sf(sf_addr + MT * 512));
#pragma unroll
          for (int m = 0; m < MT; ++m)
            if (m < mt_here) tmem_cp_sf(sfa_t + 4 * m, make_desc_sf(sf_addr + m * 512));
          // K step outside, tile inside: consecutive MMAs go to different accumulators, so one does not wait
          // for the one before it to leave the pipe (an MMA that adds to the accumulator of the MMA just
          // before it starts only when that one has finished)
#pragma unroll
          for (uint32_t k = 0; k < 4; ++k) {
#pragma unroll
            for (int m = 0; m < MT; ++m) {
              if (m < mt_here)
                mma_mx(d_tmem + m * BN, make_desc_sw128(a_addr + m * S::A_TILE) + 2 * k, bdesc + 2 * k,
                       idesc | (k << 29) | (k << 4), sfa_t + 4 * m, sfb_t, (it > 0 || k > 0) ? 1u : 0u);
            }
          }
          mma_commit(&empty_bar[s]);
        }
        if (ok) {
          mma_commit(&accf_bar[buf]);
          if (p.prof) {
            // when does the tensor core finish what was issued?  (an observer's wait does not consume the phase)
            p.prof[blockIdx.x * 8 + 5] = (long long)globaltimer_ns();
            mbar_wait(&accf_bar[buf], (ait / NACC) & 1, ab, p.status, 7);
            p.prof[blockIdx.x * 8 + 2] = (long long)globaltimer_ns();
          }
          ++ait;
        }
      }
      if (p.prof) {
        // cycles this CTA's MMA thread waited for operands / for a free accumulator, and its whole loop
        p.prof[blockIdx.x * 8 + 1] = w_full;
        (void)w_acc;
        p.prof[blockIdx.x * 8 + 3] = clock64() - t_begin;
      }
    }
  } else if (warp >= 6) {
    // ------------------------------ copy warps: weight nibbles + exponents ------------------------------
    const int ct = (warp - 6) * 32 + lane;        // 0..255
    const int r = ct >> 1, hf = ct & 1;           // weight row of the tile, which 64 values of the stage
    const uint8_t* sfb_base = reinterpret_cast<const uint8_t*>(p.b_scale);
    int cit = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < ntiles && ok; u += gridDim.x) {
      MX_TILE(u)
      (void)tile_a;
      // exponents: threads 0..127 take the weight rows, threads 128..128+BN-1 the token rows
      const uint8_t* sf_p = nullptr;
      const float* sf_f[MT];                // AKIND 1: f32 scales that are powers of two (a weight thread: one per tile)
#pragma unroll
      for (int m = 0; m < MT; ++m) sf_f[m] = nullptr;
      long long sf_fstep = 0;
      if (AKIND == 0) {
        if (ct < 128) {
          if (a_row0 + ct < tc.ra_end) sf_p = p.aq_scale + (long long)(a_row0 + ct) * p.aq_sld;
        } else if (ct - 128 < BN) {
          if (b_row0 + (ct - 128) < tc.rb_end) sf_p = sfb_base + (long long)(b_row0 + ct - 128) * p.b_ld;
        }
      } else {
        if (ct < 128) {
          // one scale per 128 x 128 weight block: [row block, K block]
          sf_fstep = 1;
#pragma unroll
          for (int m = 0; m < MT; ++m)
            if (m < mt_here && a_row0 + m * 128 + ct < tc.ra_end) sf_f[m] = p.a_scale + (long long)((a_row0 >> 7) + m) * p.a_ld;
        } else if (ct - 128 < BN) {
          // activations: one scale per token per 128 values, stored transposed [K block, token]
          if (b_row0 + (ct - 128) < tc.rb_end) { sf_f[0] = p.b_scale + (b_row0 + ct - 128); sf_fstep = p.b_ld; }
        }
      }
      const int sf_row = ct < 128 ? ct : ct - 128;
      // the token block follows the MT weight blocks
      const uint32_t sf_off = (ct < 128 ? 0u : (uint32_t)MT * 512u) + (uint32_t)(sf_row & 31) * 16u + (uint32_t)(sf_row >> 5) * 4u;
      auto fetch_sf = [&](int it, int m) -> uint32_t {
        const int kb = kb_begin + it;
        if (AKIND == 0) return sf_p ? __ldg(reinterpret_cast<const uint32_t*>(sf_p + kb * 4)) : 0u;
        // the exponent field of a power-of-two f32, replicated over the four 32-value sub-blocks
        return sf_f[m] ? ((__float_as_uint(__ldg(sf_f[m] + (long long)kb * sf_fstep)) >> 23) & 0xFFu) * 0x01010101u : 0u;
      };
      // the exponent words of the next AHEAD stages are held in registers: one word per thread, tile and stage
      uint32_t sfq[MT][AHEAD];
#pragma unroll
      for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int d = 0; d < AHEAD; ++d) sfq[m][d] = d < nkb ? fetch_sf(d, m) : 0u;
      for (int it0 = 0; it0 < nkb && ok; it0 += AHEAD) {
#pragma unroll
        for (int d = 0; d < AHEAD; ++d) {
          const int it = it0 + d;
          if (it >= nkb) break;
          const int s = cit % STAGES;
          const uint32_t ph = (cit / STAGES) & 1;
          ++cit;
          uint8_t* sa = smem + s * S::STAGE_BYTES;
          if (AKIND == 0) {
            // this stage's nibbles have landed in the staging buffer (which also means the stage is free:
            // the producer only refills a stage the tensor core has released)
            if (!mbar_wait(&raw_bar[s], ph, ab, p.status, 6)) { ok = false; break; }
            const uint4* raw = reinterpret_cast<const uint4*>(sa + S::A_BYTES + S::B_BYTES + S::SF_BYTES + r * 64 + hf * 32);
            const uint4 q0 = raw[0], q1 = raw[1];
            // 16 nibbles (8 bytes) per 16-byte chunk, the other 8 bytes are padding
            *reinterpret_cast<uint4*>(sa + sw128_offset(r, hf * 4 + 0)) = make_uint4(q0.x, q0.y, 0u, 0u);
            *reinterpret_cast<uint4*>(sa + sw128_offset(r, hf * 4 + 1)) = make_uint4(q0.z, q0.w, 0u, 0u);
            *reinterpret_cast<uint4*>(sa + sw128_offset(r, hf * 4 + 2)) = make_uint4(q1.x, q1.y, 0u, 0u);
            *reinterpret_cast<uint4*>(sa + sw128_offset(r, hf * 4 + 3)) = make_uint4(q1.z, q1.w, 0u, 0u);
          } else {
            if (!mbar_wait(&empty_bar[s], ph ^ 1, ab, p.status, 6)) { ok = false; break; }
          }
          if (ct < 128 + BN) {
#pragma unroll
            for (int m = 0; m < MT; ++m)
              if (m == 0 || ct < 128) *reinterpret_cast<uint32_t*>(sa + S::A_BYTES + S::B_BYTES + m * 512 + sf_off) = sfq[m][d];
          }
          if (it + AHEAD < nkb) {
#pragma unroll
            for (int m = 0; m < MT; ++m) sfq[m][d] = fetch_sf(it + AHEAD, m);
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&full_bar[s]);
        }
      }
    }
  } else {
    // ------------------------------ epilogue warps ------------------------------
    const int quarter = warp & 3;
    const uint32_t tw = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const int li = quarter * 32 + lane;
    int ait = 0, nst = 0;
    bool ok = true;
    long long w_accf = 0;
    long long tq[4] = {0, 0, 0, 0};      // cycles in: tensor-memory loads, staging, barrier, global stores
    __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(smem + S::EPI_OFFSET);
    const bool store_t = store_t_ok<CH>(p);
    // This code runs once or a few times per launch, so its size is its cost (every line of it is fetched
    // cold): the loops over a unit's tiles and column chunks are kept rolled and share one body.
    for (int u = blockIdx.x; u < ntiles && ok; u += gridDim.x) {
      MX_TILE(u)
      (void)tile_a;
      // split units write their partial tile to the workspace [split][unit][tile of the unit][column][row]
      const int trem = tile_ - n_full;
      float* mine = nsp > 1 ? p.ws + ((long long)split_ * nrem + trem) * (MT * 128 * BN) : nullptr;
      const int buf = ait % NACC;
      if (nkb > 0) {
        const long long t0 = p.prof ? clock64() : 0;
        ok = mbar_wait(&accf_bar[buf], (ait / NACC) & 1, ab, p.status, 5);
        if (!ok) break;
        if (p.prof) w_accf += clock64() - t0;
        tc_fence_after();
      }
      // pass 0: the accumulators, to the output (whole units) or the workspace (split units);
      // pass 1 (the split that arrived last on the unit's counter): the sum of all partials, in split order
      for (int pass = 0; pass < 2; ++pass) {
        if (pass == 1) {
          if (nkb > 0) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acce_bar[buf]);
            ++ait;
          }
          if (nsp == 1) break;
          epi_bar(128);
          if (threadIdx.x == 64) {
            __threadfence();
            const int prev = atomicAdd(&p.counters[trem], 1);
            const int last = (prev == splits - 1);
            if (last) p.counters[trem] = 0;      // the counter is left at zero
            *s_last = last;
            __threadfence();
          }
          epi_bar(128);
          const int last = *s_last;
          epi_bar(128);                            // s_last may be rewritten by the next unit
          if (!last) break;
        }
        const long long sstride = (long long)nrem * (MT * 128 * BN);
#pragma unroll 1
        for (int mc = 0; mc < mt_here * NCH; ++mc) {
          const int m = mc / NCH, c = mc % NCH;
          const int i = a_row0 + m * 128 + li;
          float v[CH];
#pragma unroll
          for (int e = 0; e < CH; ++e) v[e] = 0.f;
          if (pass == 0) {
            const long long q0 = p.prof ? clock64() : 0;
            if (nkb > 0) {
              uint32_t rr[CH];
              if constexpr (CH == 32)
                tmem_ld32(tw + buf * ACC_COLS + m * BN + c * CH, *reinterpret_cast<uint32_t(*)[32]>(rr));
              else
                tmem_ld16(tw + buf * ACC_COLS + m * BN + c * CH, *reinterpret_cast<uint32_t(*)[16]>(rr));
              tmem_ld_wait();
#pragma unroll
              for (int e = 0; e < CH; ++e) v[e] = __uint_as_float(rr[e]);
            }
            if (p.prof) tq[0] += clock64() - q0;
            if (nsp > 1) {
              if (i < tc.ra_end) {
#pragma unroll
                for (int e = 0; e < CH; ++e) mine[(m * BN + c * CH + e) * 128 + li] = v[e];
              }
              continue;
            }
          } else if (i < tc.ra_end) {
            const float* base = p.ws + (long long)trem * (MT * 128 * BN) + (m * BN + c * CH) * 128 + li;
#pragma unroll 2
            for (int sp = 0; sp < splits; ++sp) {
              float t[CH];
#pragma unroll
              for (int e = 0; e < CH; ++e) t[e] = __ldcg(base + sp * sstride + e * 128);
#pragma unroll
              for (int e = 0; e < CH; ++e) v[e] += t[e];
            }
          }
          if (store_t)
            store_chunk_t<CH>(p, tc, a_row0 + m * 128, li, b_row0 + c * CH, v, stage, (nst++) & 1, p.prof ? tq : nullptr);
          else
            store_chunk_slow<CH>(p, tc, i, b_row0 + c * CH, v);
        }
      }
    }
    if (p.prof && threadIdx.x == 64) {
      p.prof[blockIdx.x * 8 + 7] = w_accf;
      for (int q = 0; q < 4; ++q) p.prof[(148 + blockIdx.x) * 8 + q] = tq[q];
    }
  }
#undef MX_TILE

  tc_fence_before();
  if (p.prof && threadIdx.x == 64) p.prof[blockIdx.x * 8 + 6] = (long long)globaltimer_ns();   // epilogue done
  __syncthreads();
  if (warp == 1) {
    if (ab->flag) {
      for (int t = 0; t < 64; ++t) __nanosleep(2000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// How a dense launch is cut into units of work.  Whole rounds of the SMs take units of `mt` tiles over all
// of K; what is left (all of the tiles when there are fewer than SMs) goes as units of `rem_mt` tiles cut
// `splits` ways along K so the whole chip streams weights.
struct MxPlan {
  int mt, rem_mt, splits, n_full, nrem;
  double cost;
};

// Cost of a plan in KB an SM pulls through L2 on its critical path: a stage of a unit with m tiles moves
// m * 16 KB of weights and the token tile; every unit pays a pipeline fill; split units pay for writing
// their partial tile and the last arriver for reading all of them back (latency bound: one batch of loads
// per 32 columns, tile and split).
MxPlan plan_mx(int tiles_a, int nkb, int bn, int max_mt, const LkGemmArgs& a) {
  const double FILL = 60.0, BATCH = 20.0;
  MxPlan best{1, 1, 1, tiles_a, 0, 1e30};
  auto stage = [&](int m) { return m * 16.0 + bn / 8.0; };
  for (int mt = 1; mt <= max_mt; ++mt) {
    if (a.mt > 0 && mt != a.mt && !(a.mt > max_mt && mt == max_mt)) continue;
    const int rounds = tiles_a / (148 * mt);
    const int n_full = nkb > 8 ? rounds * 148 : (tiles_a + mt - 1) / mt;
    const int left = tiles_a - n_full * mt;
    const double t_full = (n_full + 147) / 148 * (nkb * stage(mt) + FILL);
    if (left <= 0) {
      if (t_full < best.cost) best = MxPlan{mt, 1, 1, n_full, 0, t_full};
      continue;
    }
    for (int rmt = 1; rmt <= mt; ++rmt) {
      if (a.rem_mt > 0 && rmt != a.rem_mt && !(a.rem_mt > mt && rmt == mt)) continue;
      const int nrem = (left + rmt - 1) / rmt;
      for (int sp = 1; sp <= 16; ++sp) {
        if (a.splits > 0 && sp != a.splits) continue;
        const int kbs = (nkb + sp - 1) / sp;
        if (sp > 1) {
          if (kbs < 4 || (long long)kbs * (sp - 1) >= nkb) continue;
          if (!a.ws || !a.counters || (long long)nrem * sp * mt * 128 * bn > a.ws_floats || nrem > a.n_counters) continue;
        }
        const int waves = (nrem * sp + 147) / 148;
        double t = t_full + waves * (kbs * stage(rmt) + FILL);
        if (sp > 1) t += rmt * bn * 0.5 + rmt * ((bn + 31) / 32) * sp * BATCH;
        if (t < best.cost) best = MxPlan{mt, rmt, sp, n_full, nrem, t};
      }
    }
  }
  return best;
}

template <int BN, int AKIND, int MT>
constexpr int mx_stages() {
  const int stage = MxSmem<BN, 1, AKIND, MT>::STAGE_BYTES;
  const int n = (227 * 1024 - 1536 - MxSmem<BN, 1, AKIND, MT>::EPI_BYTES) / stage;
  return n > 8 ? 8 : n;
}

template <int BN, int AKIND, int MT>
int launch_mx(const LkGemmArgs& a, const GemmParams& p0, const MxPlan& plan, cudaStream_t st) {
  constexpr int STAGES = mx_stages<BN, AKIND, MT>();
  static_assert(STAGES >= 3, "pipeline depth");
  using S = MxSmem<BN, STAGES, AKIND, MT>;
  CUtensorMap tmA, tmB;
  memset(&tmA, 0, sizeof(tmA));
  int rc = lkh::make_tmap_2d(&tmB, a.B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)a.Rb, (uint64_t)a.K,
                             (uint64_t)a.ldb, BN, 128);
  if (rc) return rc;
  if (AKIND == 1) {
    if (a.a_tiled)
      rc = lkh::make_tmap_2d(&tmA, a.A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1,
                             (uint64_t)((a.Ra + 127) / 128) * ((a.K + 127) / 128) * 128, 128, 128, 128, 128);
    else
      rc = lkh::make_tmap_2d(&tmA, a.A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)a.Ra, (uint64_t)a.K,
                             (uint64_t)a.lda, 128, 128);
  } else {
    // the packed nibbles as plain bytes: 128 rows x 64 bytes (128 values) per stage, no swizzle
    rc = lkh::make_tmap_2d_plain(&tmA, a.aq, (uint64_t)a.Ra, (uint64_t)(a.K >> 1), (uint64_t)a.aq_ld, 128, 64);
  }
  if (rc) return rc;
  auto kern = gemm_mx_kernel<BN, STAGES, AKIND, MT>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  GemmParams q = p0;
  const bool grouped = a.g_rows_per_expert > 0;
  q.tiles_a = grouped ? (a.g_rows_per_expert + 127) / 128 : (a.Ra + 127) / 128;
  q.tiles_b = grouped ? a.g_max_tiles : (a.Rb + BN - 1) / BN;
  q.splits = plan.splits;
  q.n_full = plan.n_full;
  q.nrem = plan.nrem;
  q.rem_mt = plan.rem_mt;
  q.ws = a.ws;
  q.counters = a.counters;
  const long long units = grouped ? (long long)q.tiles_a * q.tiles_b : (long long)plan.n_full + (long long)plan.nrem * plan.splits;
  const unsigned grid = (unsigned)(units < 148 ? units : 148);
  lkh::launch_pdl(kern, dim3(grid), dim3(MX_THREADS), S::TOTAL, st, tmA, tmB, q);
  lkh::count_launch();
  return lkh::launch_status();
}

template <int BN, int AKIND>
int launch_mx_mt(const LkGemmArgs& a, const GemmParams& p, cudaStream_t st) {
  const bool grouped = a.g_rows_per_expert > 0;
  const int tiles_a = grouped ? (a.g_rows_per_expert + 127) / 128 : (a.Ra + 127) / 128;
  const int tiles_b = grouped ? a.g_max_tiles : (a.Rb + BN - 1) / BN;
  const int nkb = (a.K + 127) / 128;
  if (grouped) return launch_mx<BN, AKIND, 1>(a, p, MxPlan{1, 1, 1, tiles_a * tiles_b, 0, 0.0}, st);
  if (AKIND == 0 || tiles_b > 1) {
    // single tiles; several token tiles: the unit list is [weight tile][token tile]
    MxPlan pl = plan_mx(tiles_a * tiles_b, nkb, BN, 1, a);
    return launch_mx<BN, AKIND, 1>(a, p, pl, st);
  }
  if constexpr (AKIND == 1) {
    const MxPlan pl = plan_mx(tiles_a, nkb, BN, 3, a);
    switch (pl.mt) {
      case 3: return launch_mx<BN, 1, 3>(a, p, pl, st);
      case 2: return launch_mx<BN, 1, 2>(a, p, pl, st);
      default: return launch_mx<BN, 1, 1>(a, p, pl, st);
    }
  }
  return LKH_BAD_ARG;
}

template <int AKIND>
int dispatch_mx(const LkGemmArgs& a, const GemmParams& p, int bn, cudaStream_t st) {
  switch (bn) {
    case 16: return launch_mx_mt<16, AKIND>(a, p, st);
    case 32: return launch_mx_mt<32, AKIND>(a, p, st);
    case 64: return launch_mx_mt<64, AKIND>(a, p, st);
    case 128: return launch_mx_mt<128, AKIND>(a, p, st);
    default: return LKH_BAD_ARG;
  }
}

}  // namespace

// Block-scaled GEMM with MXFP4 weights on the M side (fields of LkGemmArgs: `aq` = nibbles with row
// pitch `aq_ld` bytes, `aq_scale` = E8M0 exponents with row pitch `aq_sld` bytes, a multiple of 4 and
// zero-padded to 4 * ceil(K / 128)) and e4m3 token rows on the N side (`B`, row pitch `ldb` bytes;
// `b_scale` = their E8M0 exponents as bytes, row pitch `b_ld`, padded the same way).  K % 32 == 0.
LK_API int lk_gemm_mx(const LkGemmArgs* args, void* stream) {
  const LkGemmArgs& a = *args;
  if (!a.B || !a.b_scale || !a.out || a.Ra <= 0 || a.Rb <= 0 || a.K <= 0) return LKH_BAD_ARG;
  const int nkb = (a.K + 127) / 128;
  const bool fp4 = a.aq_fmt != 0;
  if ((a.K & 31) || (a.ldb & 15)) return LKH_BAD_ARG;
  if (fp4) {
    if (!a.aq || !a.aq_scale || (a.aq_ld & 15) || (a.aq_sld & 3) || (a.b_ld & 3) || a.aq_sld < nkb * 4 ||
        a.b_ld < nkb * 4 || (reinterpret_cast<uintptr_t>(a.aq) & 15) || (reinterpret_cast<uintptr_t>(a.aq_scale) & 3) ||
        (reinterpret_cast<uintptr_t>(a.b_scale) & 3))
      return LKH_BAD_ARG;
  } else {
    // e4m3 weights [Ra, K] with one power-of-two f32 scale per 128 x 128 block (a_scale [Ra / 128, a_ld]),
    // activations with one power-of-two f32 scale per token per 128 values, transposed (b_scale [K / 128, b_ld])
    if (!a.A || !a.a_scale || (a.lda & 15) || a.a_mode != SCALE_WBLOCK || a.b_mode != SCALE_ACT_T ||
        a.g_rows_per_expert > 0)
      return LKH_BAD_ARG;
  }
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.Ra = a.Ra; p.Rb = a.Rb; p.K = a.K;
  p.out_sa = a.out_sa; p.out_sb = a.out_sb;
  p.out = a.out; p.out_fp32 = a.out_fp32;
  p.bias = a.bias; p.bias_on_a = a.bias_on_a;
  p.residual = reinterpret_cast<const __nv_bfloat16*>(a.residual);
  p.a_scale = a.a_scale; p.a_ld = a.a_ld;
  p.b_scale = a.b_scale; p.b_ld = a.b_ld;
  p.status = a.status;
  p.a_tiled = a.a_tiled;
  p.prof = a.prof;
  p.aq = reinterpret_cast<const uint8_t*>(a.aq); p.aq_scale = reinterpret_cast<const uint8_t*>(a.aq_scale);
  p.aq_ld = a.aq_ld; p.aq_sld = a.aq_sld;
  p.g_tile_expert = a.g_tile_expert; p.g_tile_row0 = a.g_tile_row0; p.g_tile_rows = a.g_tile_rows;
  p.g_ntiles = a.g_ntiles; p.g_rows_per_expert = a.g_rows_per_expert;
  if (a.g_rows_per_expert > 0 && (!a.g_tile_expert || !a.g_tile_row0 || !a.g_tile_rows || !a.g_ntiles ||
                                  a.g_max_tiles <= 0))
    return LKH_BAD_ARG;
  int bn = a.bn;
  if (bn <= 0) {
    bn = 16;
    while (bn < a.Rb && bn < 128) bn *= 2;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return fp4 ? dispatch_mx<0>(a, p, bn, st) : dispatch_mx<1>(a, p, bn, st);
}
