// C interface of libloken_host.so: GGUF reader / writer, block codecs, the CPU decode path,
// the paged-KV allocator hot path and the wire codec.  Plain C so ctypes can bind it.
#pragma once
#include <stdint.h>

#define LKH_API extern "C" __attribute__((visibility("default")))

// ---- GGUF reader (gguf.cpp) ----
LKH_API void* lkg_open(const char* path, char* err, int err_cap);
LKH_API void lkg_close(void* h);
LKH_API int lkg_version(void* h);
LKH_API long long lkg_alignment(void* h);
LKH_API long long lkg_n_tensors(void* h);
LKH_API long long lkg_n_kv(void* h);
LKH_API int lkg_tensor_info(void* h, long long i, char* name, int cap, long long* dims, int* n_dims, int* type,
                            long long* nbytes);
LKH_API const void* lkg_tensor_data(void* h, long long i);
LKH_API int lkg_tensor_advise(void* h, long long i, int advice);
LKH_API int lkg_kv_info(void* h, long long i, char* key, int cap, int* type, int* elem_type, long long* count);
LKH_API double lkg_kv_num(void* h, long long i, long long j);
LKH_API long long lkg_kv_int(void* h, long long i, long long j);
LKH_API long long lkg_kv_str(void* h, long long i, long long j, char* buf, long long cap);
LKH_API long long lkg_kv_array_raw(void* h, long long i, void* dst, long long cap_bytes);

// ---- GGUF writer (gguf_write.cpp) ----
LKH_API void* lkw_create(const char* path, int alignment);
LKH_API int lkw_kv_u32(void* w, const char* key, uint32_t v);
LKH_API int lkw_kv_i32(void* w, const char* key, int32_t v);
LKH_API int lkw_kv_u64(void* w, const char* key, uint64_t v);
LKH_API int lkw_kv_f32(void* w, const char* key, float v);
LKH_API int lkw_kv_bool(void* w, const char* key, int v);
LKH_API int lkw_kv_str(void* w, const char* key, const char* v, long long n);
LKH_API int lkw_kv_arr_num(void* w, const char* key, int elem_type, const void* data, long long count);
LKH_API int lkw_kv_arr_str(void* w, const char* key, const char* const* strs, const long long* lens, long long count);
// Declares a tensor; its payload is streamed later, in declaration order, by lkw_write_tensor.
LKH_API int lkw_add_tensor(void* w, const char* name, const long long* dims, int n_dims, int type);
LKH_API int lkw_begin_data(void* w);
LKH_API int lkw_write_tensor(void* w, const void* data, long long nbytes);
LKH_API int lkw_finish(void* w);

// ---- block codecs (codec_api.cpp) ----
LKH_API int lkc_block_info(int type, int* block_values, int* block_bytes);
LKH_API int lkc_dequant(int type, const void* src, float* dst, long long n, int threads);
LKH_API int lkc_quant(int type, const float* src, void* dst, long long n, int threads);
LKH_API int lkc_cpu_level(void);

// ---- CPU decode path (cpu_decode.cpp) ----
typedef struct LkCpuConfig {
  int n_layers, hidden, n_q, n_kv, head_dim, intermediate, vocab;
  int rope_dim;        // 0 = head_dim
  int rope_pairing;    // 0 adjacent lane pairs, 1 half-split
  float rope_theta, rms_eps;
} LkCpuConfig;
// threads <= 0: one per hardware thread; max_level caps the SIMD level (see lkc_cpu_level), -1 = best
LKH_API void* lkcpu_create(const LkCpuConfig* cfg, int threads, int max_level);
LKH_API void lkcpu_free(void* h);
LKH_API int lkcpu_set_inv_freq(void* h, const float* inv_freq, int n);
// roles per layer: 0 attn_norm, 1 q, 2 k, 3 v, 4 o, 5 q_norm, 6 k_norm, 7 ffn_norm, 8 gate, 9 up, 10 down,
// 11..13 q/k/v bias; layer < 0: 100 token embedding, 101 output norm, 102 lm head
LKH_API int lkcpu_set_tensor(void* h, int layer, int role, const void* data, int type);
LKH_API int lkcpu_ready(void* h);
LKH_API int lkcpu_decode(void* h, int token, int pos, float* logits);
LKH_API int lkcpu_level(void* h);
LKH_API int lkcpu_threads(void* h);
LKH_API float lkcpu_dot_q8_0(const void* x, const void* y, int nblocks, int level);
LKH_API int lkcpu_gemv_q8_0(const void* w, const float* x, float* out, int N, int K, int threads, int level);
// (token, expert) pairs of a mixture layer on the host cores over expert stacks in the device plane layouts
// (fmt 0 bf16, 1 Q8_0, 2 Q6_K, 3 Q4_K, 4 MXFP4; scale pitches in bytes, 0 = the format's own row size):
// out[t] += w * down_e(glu(gate_up_e(x[t]))).
LKH_API int lkcpu_moe_pairs(int fmt_gu, const void* gu_codes, const void* gu_scales, int fmt_dn, const void* dn_codes,
                            const void* dn_scales, const float* gu_bias, const float* dn_bias, int H, int I,
                            const float* x, const int* pair_tok, const int* pair_expert, const float* pair_w, int n_pairs,
                            int glu_mode, float alpha, float limit, float* out, int threads, int max_level,
                            long long gu_scale_pitch, long long dn_scale_pitch);
LKH_API int lkcpu_gemv_any(int type, const void* w, const float* x, float* out, int N, int K, int threads, int level);

// ---- wire codec (wire.cpp) ----
LKH_API long long lkwire_header_bytes(int rank);
LKH_API long long lkwire_payload_bytes(int dtype, long long n);
LKH_API long long lkwire_encode_header(uint8_t* dst, long long cap, int kind, unsigned long long request_id,
                                       unsigned layer, int dtype, int rank, const unsigned* dims,
                                       unsigned long long payload_bytes);
LKH_API long long lkwire_decode_header(const uint8_t* src, long long n, int* kind, unsigned long long* request_id,
                                       unsigned* layer, int* dtype, int* rank, unsigned* dims,
                                       unsigned long long* payload_bytes);
LKH_API long long lkwire_pack(int dtype, const float* src, long long n, uint8_t* dst, long long cap);
LKH_API long long lkwire_unpack(int dtype, const uint8_t* src, long long nbytes, float* dst, long long n);
