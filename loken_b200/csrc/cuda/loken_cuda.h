// C interface of libloken_cuda.so.  Every launcher takes raw device pointers and the CUDA
// stream to launch on, allocates nothing, and returns 0 when the kernel was launched
// (negative: refused before launch, positive: CUDA runtime error code).
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- tcgen05 GEMM: C[i, j] = sum_k A[i, k] * B[j, k] (gemm_tc.cuh) -----------------------
typedef struct LkGemmArgs {
  int kind;               // 0 = bf16 operands, 1 = e4m3 operands with block scales
  const void* A;          // [Ra, K], row pitch lda elements: rows on the MMA M side
  const void* B;          // [Rb, K], row pitch ldb elements: rows on the MMA N side
  int Ra, Rb, K;
  long long lda, ldb;
  void* out;              // bf16, or fp32 when out_fp32
  long long out_sa, out_sb;
  int out_fp32;
  const float* bias;      // optional
  int bias_on_a;
  const void* residual;   // optional bf16, same strides as out
  const float* a_scale;   // fp8 kind: see a_mode
  int a_mode;             // 0 none, 1 weight blocks [(row/128), kb], 2 activations transposed [kb, row]
  long long a_ld;
  const float* b_scale;
  int b_mode;
  long long b_ld;
  int bn;                 // N tile (16..256, power of two), 0 = choose from Rb
  int splits;             // split-K factor (needs ws + counters when > 1)
  float* ws;
  long long ws_floats;
  int* counters;
  int n_counters;
  int* status;            // device error word (may be null)
  const void* symm_view;  // optional lk::SymmView: sum the output over its ranks inside the epilogue
  // quantised A (weights on the M side), expanded to bf16 inside the kernel (dequant.cuh):
  // 0 none, 1 int8 + f16 scale/32, 2 int8 + f16 scale/16, 3 nibbles + (scale, min)/32, 4 MXFP4
  int aq_fmt;
  const void* aq;         // code plane, row pitch aq_ld bytes
  const void* aq_scale;   // scale plane, row pitch aq_sld bytes
  long long aq_ld, aq_sld;
  // grouped (mixture of experts): A = E stacked matrices of g_rows_per_expert rows, B = token rows
  // sorted by expert, N tiles listed on the device
  int g_rows_per_expert;  // 0 = not grouped
  int g_max_tiles;        // capacity of the tile list (bounds the grid)
  const int* g_tile_expert;
  const int* g_tile_row0;
  const int* g_tile_rows;
  const int* g_ntiles;
  // lk_gemm_mx, dense e4m3 weights: weight tiles per unit of work in the whole rounds / in the K-split
  // remainder (0 = the launcher's cost model chooses; `splits` above likewise)
  int mt, rem_mt;
  // e4m3 weights stored tile-major: [ceil(Ra / 128)][ceil(K / 128)][128 rows][128 bytes], zero padded
  int a_tiled;
  // lk_gemm_mx, optional: int64 [296 x 8].  Row c < 148 (CTA c): cycles the producer waited for a free
  // stage; cycles the MMA thread waited for operands; global-timer ns when the last unit's MMAs had
  // completed; cycles of the MMA thread's whole loop; global-timer ns at the CTA's start, when the last
  // unit's MMAs were issued, and at the end of the epilogue; cycles the epilogue waited for accumulators.
  // Row 148 + c: cycles the epilogue spent in tensor-memory loads, staging, its barrier, global stores.
  long long* prof;
} LkGemmArgs;

int lk_gemm_tc(const LkGemmArgs* args, void* stream);
unsigned long long lk_launch_count(void);
// Block-scaled GEMM (gemm_mx.cu): MXFP4 weights on the M side (`aq` nibbles, `aq_scale` E8M0 exponents per 32
// values), e4m3 token rows with E8M0 exponents on the N side (`B`, `b_scale` as bytes, pitch `b_ld`); scales
// applied by `tcgen05.mma.kind::mxf8f6f4.block_scale`.
int lk_gemm_mx(const LkGemmArgs* args, void* stream);
// bf16 rows -> e4m3 + one E8M0 exponent per 32 values, fused with a row gather or a GLU (mx_quant.cu)
int lk_quant_mx8(const void* x, long long ldx, int rows, int K, int mode, const int* pair_row, int kdiv,
                 int glu_mode, float alpha, float limit, void* out, long long ldo, void* sf, long long sf_ld,
                 void* stream);

// ---- row kernels (elementwise.cu) -------------------------------------------------------
int lk_embed_bf16(const int* tokens, const void* table, void* out, int T, int H, int vocab, float scale,
                  void* stream);
int lk_add_rmsnorm(void* x, const void* delta, const float* delta_f32, const float* w, float eps, int T, int H,
                   void* out_bf16, void* out_fp8, float* scales_t, long long scale_ld, int write_x, void* stream);
int lk_glu(const void* gate_up, long long ld_in, int T, int I, int mode, float alpha, float limit, void* out_bf16,
           void* out_fp8, float* scales_t, long long scale_ld, void* stream);
int lk_quant_fp8(const void* x, long long ld_in, int T, int K, void* out, float* scales_t, long long scale_ld,
                 void* stream);
int lk_add_bf16(const void* a, const void* b, void* out, long long n, void* stream);

// ---- fused q/k norm + RoPE + paged KV write; cache gather for prefill (rope_kv.cu) --------
int lk_rope_kv(const void* qkv, long long ld, const int* pos, const int* slots, int T, int n_q, int n_kv, int hd,
               const float* q_norm_w, const float* k_norm_w, float eps, const float* inv_freq, int rope_dim,
               int pairing, float mscale, void* q_out, void* k_cache, void* v_cache, void* k_scale, void* v_scale,
               long long num_slots, int kv_q8, int* status, void* stream);
// The same with the q / k norm taken over the token's whole projection (OLMoE); `rinv` is [T, 2] f32 scratch.
int lk_rope_kv_wide(const void* qkv, long long ld, const int* pos, const int* slots, int T, int n_q, int n_kv, int hd,
                    const float* q_norm_w, const float* k_norm_w, float eps, const float* inv_freq, int rope_dim,
                    int pairing, float mscale, void* q_out, void* k_cache, void* v_cache, void* k_scale, void* v_scale,
                    long long num_slots, int kv_q8, int* status, float* rinv, void* stream);
// Context shift: cache positions move from `src` to `dst` slots (no overlap); key i is turned by delta[i]
// positions on the way, values are copied.
// What the activations of a GEMV are computed from, and a residual update it applies on the side.
typedef struct {
  int mode;                 // 0: the rows of x; 1: RMSNorm(x + delta) * gamma; 2: gated unit of x = [gate | up] (2K wide)
  const void* delta;        // mode 1: bf16 [M, K] update still pending on x (row pitch ldd elements), or null
  long long ldd;
  const float* gamma;       // mode 1: [K]
  float eps;
  int glu_mode;             // mode 2: 0 silu(g) * u; 1 the clamped form (alpha, limit)
  float glu_alpha, glu_limit;
  void* upd_x;              // bf16 [M, upd_cols]: upd_x += upd_delta (rounded once), applied by one CTA; or null
  const void* upd_delta;
  long long upd_ldx, upd_ldd;
  int upd_cols;
  void* prof;               // measurement hook: int64 [CTAs][8] time stamps of the streaming form, or null
} LkGemvPre;

// Quantised GEMV for 1..8 token rows: int8 activations (quantised per 32 values inside the kernel) and
// dp4a over the stored codes.  fmt: 1 Q8_0, 2 Q6_K, 3 Q4_K planes of ops/quant.py.
int lk_gemv_q(int fmt, const void* codes, long long c_ld, const void* scales, long long s_ld, const void* x,
              long long ldx, int M, int N, int K, const float* bias, void* out, long long ldo, int out_fp32,
              const LkGemvPre* pre, int* status, void* stream);
// 0: every GEMV on the register form; 1 (default): the streaming form (bulk-copy ring) where the shape allows;
// 3: the same plus L2 hints for the rows the ring does not hold yet.
void lk_gemv_q_stream(int on);
// The same planes decoded to bf16 out [rows, K], row pitch ldo elements: the operand of prompt-sized GEMMs.
int lk_dequant_q(int fmt, const void* codes, long long c_ld, const void* scales, long long s_ld, void* out,
                 long long ldo, int rows, int K, void* stream);
// Expert slots on the streaming GEMV: slot s multiplies row s / x_div of x by expert slot_expert[s] - e_lo of a stack
// of n_experts [N, K] matrices (contiguous planes) and writes row s of out [slots, N]; expert ids are read on the
// device.  dry != 0 only answers whether the shape is taken (0) or not (bad argument).
int lk_gemv_q_slots(int fmt, const void* codes, const void* scales, const void* x, long long ldx, int slots, int x_div,
                    const int* slot_expert, int e_lo, int n_experts, int N, int K, const float* bias, void* out,
                    long long ldo, const LkGemvPre* pre, int* status, int dry, void* stream);
// Embedding gather from a quantised table (the same planes): rows tokens[0 .. T) decoded to bf16 out [T, H].
int lk_embed_q(int fmt, const int* tokens, const void* codes, long long c_ld, const void* scales, long long s_ld,
               void* out, int T, int H, int vocab, float scale, void* stream);
int lk_kv_shift(void* k_cache, void* v_cache, void* k_scale, void* v_scale, const int* src, const int* dst,
                const int* delta, int n, int n_kv, int hd, const float* inv_freq, int rope_dim, int pairing,
                long long num_slots, int kv_q8, int* status, void* stream);
int lk_kv_gather(const void* k_cache, const void* v_cache, const void* k_scale, const void* v_scale, int kv_q8,
                 int n_kv, int hd, const int* block_table, int max_blocks, int block_size, const int* seq_of_tile,
                 const int* tile_tok0, int n_tiles, const int* kv_len, const int* dst_off, void* k_out,
                 void* vt_out, long long ld_tok, long long num_slots, void* stream);

// ---- paged flash decode (attn_decode.cu) ---------------------------------------------------
typedef struct LkDecodeArgs {
  const void* q;            // bf16 [rows, n_q, hd]
  const void* k_cache;      // q8: int8 [slots, n_kv, hd]; else bf16
  const void* v_cache;
  const void* k_scale;      // q8: f16 [slots, n_kv, hd/32]
  const void* v_scale;
  const int* block_table;   // [n_seqs, max_blocks]
  const int* row_seq;       // optional [rows]: block-table row of each query row
  const int* seq_lens;      // [rows]: keys visible to the row
  const float* sinks;       // optional [n_q]
  void* out;                // bf16 [rows, n_q*hd] (optional when out_fp8)
  void* out_fp8;            // optional e4m3 [rows, n_q*hd], hd == 128 only
  float* out_scales_t;      // [n_q, scale_ld]
  long long scale_ld;
  float* ws;
  long long ws_floats;
  int* counters;
  int n_counters;
  int* status;
  long long num_slots;
  int rows, n_q, n_kv, hd, max_blocks, block_size, window, kv_q8, nsplit;
  float scale;
  float* parts_out;         // lk_attn_decode only, optional f32 [rows, n_q, hd + 2]: instead of the attention, what
                            // this cache contributes to it: the values weighed by exp2(score - max) (not divided),
                            // then the maximum (log2 units of the scaled scores) and the sum of the weights;
                            // parts of several caches merge into the attention over all of them
} LkDecodeArgs;
long long lk_attn_decode_ws_floats(int rows, int n_q, int n_kv, int hd, int nsplit);
int lk_attn_decode(const LkDecodeArgs* args, void* stream);
// TMA-staged variant: head_dim 128, q8 cache, 16-token pages (attn_decode_tma.cu)
int lk_attn_decode_tma(const LkDecodeArgs* args, void* stream);
// tcgen05 variant: both products on the tensor cores straight from the q8 pages (attn_decode_tc.cu)
int lk_attn_decode_tc(const LkDecodeArgs* args, void* stream);

// ---- tcgen05 flash prefill (attn_prefill.cu) -------------------------------------------------
typedef struct LkPrefillArgs {
  const void* q;          // bf16 [total_q, n_q, hd]
  const void* k;          // bf16 [total_kv_pad, n_kv, hd], sequence s at rows kv_off[s]..
  const void* vt;         // bf16 [n_kv, hd, total_kv_pad]
  void* out;              // bf16 [total_q, n_q*hd]
  const float* sinks;     // optional [n_q]
  const int* tile_seq;    // [n_tiles] sequence of each 128-row tile
  const int* tile_q0;     // [n_tiles] first query token of the tile, relative to its sequence
  const int* q_start;     // [n_seqs] first row of the sequence in q / out
  const int* q_len;       // [n_seqs]
  const int* kv_off;      // [n_seqs] first row in k (multiple of 128)
  const int* kv_len;      // [n_seqs] keys of the sequence, the last q_len of them are the queries' own
  int* status;
  int n_tiles, total_q;
  long long total_kv_pad; // multiple of 128
  int n_q, n_kv, hd, window;
  float scale;
} LkPrefillArgs;
int lk_attn_prefill(const LkPrefillArgs* args, void* stream);

// ---- sampler (sampler.cu), decode bookkeeping (step.cu) ----------------------------------------
int lk_argmax(const float* logits, long long ld, int B, int V, int* out, void* stream);
int lk_repeat_penalty(float* logits, long long ld, int B, int V, const int* recent, int L, const float* penalty,
                      void* stream);
// per-row (id, value) rules: mode 0 adds values (ban = -inf), mode 1 keeps only the listed ids; R <= 512
int lk_token_rules(float* logits, long long ld, int B, int V, const int* ids, const float* vals, const int* counts,
                   const int* modes, int R, void* stream);
// grammar masks: bits [B, words] (bit t of a row = token t allowed), rows with has[r] == 0 untouched
int lk_token_bitmask(float* logits, long long ld, int B, int V, const unsigned* bits, int words, const int* has,
                     void* stream);
int lk_sample(const float* logits, long long ld, int B, int V, const float* temperature, const int* top_k,
              const float* top_p, const float* min_p, const float* uniform, int* out, void* stream);
// 0: every row on the one-CTA sampler; 1 (default): a cluster of eight CTAs per row up to 148 rows.
void lk_sample_cluster(int on);
int lk_advance_decode(int* tokens, int* positions, int* slots, int* seq_lens, const int* sampled,
                      const int* block_table, int max_blocks, int block_size, int rows, long long num_slots,
                      int* history, int hist_ld, const int* hist_base, int* status, void* stream);

// ---- mixture of experts: routing, plan, permute, combine (moe.cu) -------------------------------
// mode: 0 softmax over the chosen logits, 1 full softmax (renorm optional), 2 sigmoid (renorm optional)
int lk_moe_route(const float* logits, long long ld, int T, int E, int k, int mode, int renorm, int* ids,
                 float* wts, void* stream);
// router GEMV + top-k in one launch (decode-size steps): h bf16 [T, ldh], w bf16 [E, H]
int lk_moe_router(const void* h, long long ldh, const void* w, const float* bias, int T, int H, int E, int k,
                  int mode, int renorm, int* ids, float* wts, float* logits_out, long long ldl, void* stream);
int lk_moe_plan(const int* ids, int P, int E_total, int e_lo, int e_cnt, int BN, int max_tiles, int* offsets,
                int* pair_row, int* tile_expert, int* tile_row0, int* tile_rows, int* ntiles, int* status,
                void* stream);
int lk_moe_permute(const void* x, long long ldx, const int* pair_row, int P, int k, int H, void* xs, long long lds,
                   void* stream);
int lk_moe_combine(const void* y, long long ldy, const int* pair_row, const float* wts, int T, int k, int H,
                   void* out, long long ldo, int accumulate, void* stream);

// ---- symmetric memory over CUDA IPC + peer-memory collectives (symm.cu) ---------------------------
// `view` points at a host copy of lk::SymmView (symm.cuh), built by the caller from the mapped heaps.
int lk_symm_alloc(long long bytes, void** out);
int lk_symm_free(void* p);
int lk_ipc_export(void* p, void* handle64);
int lk_ipc_open(const void* handle64, void** out);
int lk_ipc_close(void* p);
int lk_symm_view_size(void);
void lk_allreduce_set_mode(int mode);   /* 0 auto, 1 one-shot, 2 two-shot; the same on every rank */
int lk_allreduce_push(const void* view, void* data, int rows, int cols, long long ld, const void* residual,
                      int* status, void* stream);
// Row-parallel layer boundary in one kernel: reduce-scatter of the ranks' partial rows, residual add
// and RMSNorm on the owner of each row, (e4m3 quantise,) all-gather of the normalised rows (tp_fused.cu).
// gather: 0 = normalised rows stay on their owner, 1 = every rank receives every row.
// local: 1 = `partial` already holds the complete update of the rows this rank owns (nothing is summed
// over ranks; expert-parallel combine output), 0 = it is this rank's partial of every row.
int lk_tp_sum_norm(const void* view, const void* partial, long long ld_p, void* x, long long ld_x, const float* w,
                   float eps, int T, int H, void* out_bf16, long long ld_o, void* out_fp8, float* scales_t,
                   long long scale_ld, int gather, int local, int* status, void* stream);
// Expert-parallel dispatch / combine over peer memory (ep_moe.cu)
int lk_ep_slots(const void* view, int T, int k);
int lk_ep_dispatch(const void* view, const void* h, long long ldh, const int* ids, int T, int H, int k,
                   int n_experts, int* status, void* stream);
int lk_ep_meta(const void* view, int T, int H, int k, int n_experts, int* slot_expert, int* slot_src, int* status,
               void* stream);
int lk_ep_gather(const void* view, int T, int H, int k, int n_experts, const int* slot_expert, void* xr,
                 long long ldx, int* status, void* stream);
int lk_ep_return(const void* view, int T, int H, int k, int n_experts, const int* slot_src, const int* pair_row,
                 const void* y, long long ldy, void* stream);
int lk_ep_combine(const void* view, int T, int H, int k, int n_experts, const float* wts, void* out, long long ldo,
                  int* status, void* stream);

#ifdef __cplusplus
}
#endif
