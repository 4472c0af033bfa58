// CPU decode path: one token through a dense decoder with quantised weights on the host cores.
//
// What it restates (reference: src/inference/kernel/cpu_decode_exec.rs, src/tensor/quant_cpu/
// format/q8_0.rs, src/tensor/quant_cpu/gemv_pool.rs, src/inference/cache/cpu_q8_kv.rs):
//   * activations are quantised to Q8_0 (d = amax / 127 as f16, q = round(v / d)) before every
//     matrix product; a Q8_0 x Q8_0 row dot is per block (sum a*b as i32) * d_x * d_y, one f32
//     rounding per block; AVX-512 VNNI, AVX2 and scalar versions picked at run time, the scalar
//     one being the definition the others are tested against;
//   * Q4_K and Q6_K rows take integer dots with the same Q8_0 activation (their sub-blocks sit inside its
//     blocks of 32), AVX2 and scalar; the float formats (F16, BF16, F32) a row conversion + f32 dot;
//   * one arena of per-token scratch sized once from the model shape — no allocation per token;
//   * a persistent worker pool: workers spin briefly on a generation counter, take chunk indices
//     from a shared ticket word, and park on a condition variable when nothing arrives;
//   * the KV cache keeps Q8_0 rows per (position, kv head); scores are Q8_0 x Q8_0 dots with the
//     quantised query, values are accumulated as o += (p * d_block) * qs.
#include <atomic>
#include <condition_variable>
#include <math.h>
#include <mutex>
#include <stdlib.h>
#include <string.h>
#include <thread>
#include <vector>

#if defined(__x86_64__)
#include <immintrin.h>
#endif

#include "formats.h"
#include "loken_host.h"

using namespace lkf;

namespace {

// ------------------------------------------------------------------------------ dots
float dot_q8_scalar(const BlockQ8_0* x, const BlockQ8_0* y, int nb) {
  float acc = 0.f;
  for (int b = 0; b < nb; ++b) {
    int32_t s = 0;
    for (int i = 0; i < 32; ++i) s += (int32_t)x[b].qs[i] * (int32_t)y[b].qs[i];
    acc += (float)s * f16_to_f32(x[b].d) * f16_to_f32(y[b].d);
  }
  return acc;
}

#if defined(__x86_64__)
__attribute__((target("avx2,fma,f16c"))) float dot_q8_avx2(const BlockQ8_0* x, const BlockQ8_0* y, int nb) {
  __m256 acc = _mm256_setzero_ps();
  for (int b = 0; b < nb; ++b) {
    const __m256i a = _mm256_loadu_si256((const __m256i*)x[b].qs);
    const __m256i c = _mm256_loadu_si256((const __m256i*)y[b].qs);
    // maddubs wants unsigned x signed: |a| * sign(a)(c)
    const __m256i ax = _mm256_sign_epi8(a, a);
    const __m256i sy = _mm256_sign_epi8(c, a);
    const __m256i p16 = _mm256_maddubs_epi16(ax, sy);
    const __m256i p32 = _mm256_madd_epi16(p16, _mm256_set1_epi16(1));
    const float d = f16_to_f32(x[b].d) * f16_to_f32(y[b].d);
    // one f32 rounding per block: reduce the block's integers first
    __m128i s = _mm_add_epi32(_mm256_castsi256_si128(p32), _mm256_extracti128_si256(p32, 1));
    s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0x4E));
    s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0xB1));
    acc = _mm256_add_ps(acc, _mm256_set_ps(0, 0, 0, 0, 0, 0, 0, (float)_mm_cvtsi128_si32(s) * d));
  }
  float out[8];
  _mm256_storeu_ps(out, acc);
  return out[0];
}

__attribute__((target("avx512f,avx512bw,avx512vl,avx512vnni,avx2,fma"))) float dot_q8_vnni(const BlockQ8_0* x,
                                                                                            const BlockQ8_0* y,
                                                                                            int nb) {
  float acc = 0.f;
  for (int b = 0; b < nb; ++b) {
    const __m256i a = _mm256_loadu_si256((const __m256i*)x[b].qs);
    const __m256i c = _mm256_loadu_si256((const __m256i*)y[b].qs);
    const __m256i ax = _mm256_sign_epi8(a, a);
    const __m256i sy = _mm256_sign_epi8(c, a);
    const __m256i p32 = _mm256_dpbusd_epi32(_mm256_setzero_si256(), ax, sy);
    __m128i s = _mm_add_epi32(_mm256_castsi256_si128(p32), _mm256_extracti128_si256(p32, 1));
    s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0x4E));
    s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0xB1));
    acc += (float)_mm_cvtsi128_si32(s) * (f16_to_f32(x[b].d) * f16_to_f32(y[b].d));
  }
  return acc;
}
#endif

typedef float (*DotFn)(const BlockQ8_0*, const BlockQ8_0*, int);

DotFn pick_dot(int level) {
#if defined(__x86_64__)
  if (level >= 4) return dot_q8_vnni;
  if (level >= 2) return dot_q8_avx2;
#endif
  (void)level;
  return dot_q8_scalar;
}

// ---- K-quant rows against Q8_0 activations -----------------------------------------------------
// The activation of a product is quantised per 32 values (Q8_0), and both K formats are built from groups
// that sit inside such a block, so their row dots run on the stored integer codes as well:
//   Q4_K  sub-block s (32 values, 6-bit scale sc and minimum m against the block's d, dmin):
//           dx * (d * sc * sum(q * xq) - dmin * m * sum(xq))
//   Q6_K  two groups of 16 values (int8 scales sa, sb against d) per activation block, codes stored
//         unsigned with an offset of 32:   dx * d * (sa * (sum_a(qu * xq) - 32 sum_a(xq)) + sb * (...))
// One f32 rounding per activation block.  The scalar versions are the definitions.
// (reference: src/tensor/quant_cpu/format/{q4_k,q6_k}.rs, int8 dots of the same shape)
float dot_q4k_scalar(const BlockQ4_K* w, const BlockQ8_0* x, int nsb) {
  float acc = 0.f;
  for (int i = 0; i < nsb; ++i) {
    const float d = f16_to_f32(w[i].d), dmin = f16_to_f32(w[i].dmin);
    const uint8_t* q = w[i].qs;
    for (int j = 0; j < 4; ++j, q += 32) {
      const BlockQ8_0& xa = x[i * 8 + 2 * j];
      const BlockQ8_0& xb = x[i * 8 + 2 * j + 1];
      uint8_t sa, ma, sb, mb;
      get_scale_min_k4(2 * j, w[i].scales, &sa, &ma);
      get_scale_min_k4(2 * j + 1, w[i].scales, &sb, &mb);
      int32_t ia = 0, ib = 0, xsa = 0, xsb = 0;
      for (int l = 0; l < 32; ++l) {
        ia += (int32_t)(q[l] & 0xF) * xa.qs[l];
        ib += (int32_t)(q[l] >> 4) * xb.qs[l];
        xsa += xa.qs[l];
        xsb += xb.qs[l];
      }
      acc += f16_to_f32(xa.d) * (d * (float)sa * (float)ia - dmin * (float)ma * (float)xsa);
      acc += f16_to_f32(xb.d) * (d * (float)sb * (float)ib - dmin * (float)mb * (float)xsb);
    }
  }
  return acc;
}

float dot_q6k_scalar(const BlockQ6_K* w, const BlockQ8_0* x, int nsb) {
  float acc = 0.f;
  for (int i = 0; i < nsb; ++i) {
    const float d = f16_to_f32(w[i].d);
    for (int half = 0; half < 2; ++half) {
      const uint8_t* ql = w[i].ql + 64 * half;
      const uint8_t* qh = w[i].qh + 32 * half;
      const int8_t* sc = w[i].scales + 8 * half;
      for (int part = 0; part < 4; ++part) {            // 32 values each: one activation block
        const BlockQ8_0& xb = x[i * 8 + half * 4 + part];
        int32_t sum[2] = {0, 0};
        for (int l = 0; l < 32; ++l) {
          const int lo = (part & 1) ? ql[l + 32] : ql[l];
          const int nib = (part & 2) ? (lo >> 4) : (lo & 0xF);
          const int q = (nib | (((qh[l] >> (2 * part)) & 3) << 4)) - 32;
          sum[l / 16] += q * xb.qs[l];
        }
        acc += f16_to_f32(xb.d) * d * ((float)sc[2 * part] * (float)sum[0] + (float)sc[2 * part + 1] * (float)sum[1]);
      }
    }
  }
  return acc;
}

#if defined(__x86_64__)
__attribute__((target("avx2"))) static inline int32_t hsum_i32(__m256i v) {
  __m128i s = _mm_add_epi32(_mm256_castsi256_si128(v), _mm256_extracti128_si256(v, 1));
  s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0x4E));
  s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0xB1));
  return _mm_cvtsi128_si32(s);
}

// u8 codes times s8 activations, summed to eight i32 lanes (lanes 0-3: values 0-15, lanes 4-7: values 16-31)
__attribute__((target("avx2"))) static inline __m256i mul_sum_i32(__m256i qu, __m256i xs) {
  return _mm256_madd_epi16(_mm256_maddubs_epi16(qu, xs), _mm256_set1_epi16(1));
}

// The AVX2 versions keep eight f32 partial sums (one per i32 lane of the products) and add them up once per
// row, instead of reducing every sub-block to a scalar.
__attribute__((target("avx2,fma,f16c"))) static inline float hsum_f32(__m256 v) {
  __m128 s = _mm_add_ps(_mm256_castps256_ps128(v), _mm256_extractf128_ps(v, 1));
  s = _mm_add_ps(s, _mm_movehl_ps(s, s));
  s = _mm_add_ss(s, _mm_shuffle_ps(s, s, 1));
  return _mm_cvtss_f32(s);
}

__attribute__((target("avx2,fma,f16c"))) float dot_q4k_avx2(const BlockQ4_K* w, const BlockQ8_0* x, int nsb) {
  const __m256i m4 = _mm256_set1_epi8(0xF), one = _mm256_set1_epi8(1);
  __m256 acc = _mm256_setzero_ps();
  for (int i = 0; i < nsb; ++i) {
    const float d = f16_to_f32(w[i].d), dmin = f16_to_f32(w[i].dmin);
    const uint8_t* q = w[i].qs;
    for (int j = 0; j < 4; ++j, q += 32) {
      const BlockQ8_0& xa = x[i * 8 + 2 * j];
      const BlockQ8_0& xb = x[i * 8 + 2 * j + 1];
      uint8_t sa, ma, sb, mb;
      get_scale_min_k4(2 * j, w[i].scales, &sa, &ma);
      get_scale_min_k4(2 * j + 1, w[i].scales, &sb, &mb);
      const float dxa = f16_to_f32(xa.d), dxb = f16_to_f32(xb.d);
      const __m256i qq = _mm256_loadu_si256((const __m256i*)q);
      const __m256i va = _mm256_loadu_si256((const __m256i*)xa.qs), vb = _mm256_loadu_si256((const __m256i*)xb.qs);
      const __m256 pa = _mm256_cvtepi32_ps(mul_sum_i32(_mm256_and_si256(qq, m4), va));
      const __m256 pb = _mm256_cvtepi32_ps(mul_sum_i32(_mm256_and_si256(_mm256_srli_epi16(qq, 4), m4), vb));
      const __m256 xsa = _mm256_cvtepi32_ps(mul_sum_i32(one, va)), xsb = _mm256_cvtepi32_ps(mul_sum_i32(one, vb));
      acc = _mm256_fmadd_ps(pa, _mm256_set1_ps(dxa * d * (float)sa), acc);
      acc = _mm256_fnmadd_ps(xsa, _mm256_set1_ps(dxa * dmin * (float)ma), acc);
      acc = _mm256_fmadd_ps(pb, _mm256_set1_ps(dxb * d * (float)sb), acc);
      acc = _mm256_fnmadd_ps(xsb, _mm256_set1_ps(dxb * dmin * (float)mb), acc);
    }
  }
  return hsum_f32(acc);
}

__attribute__((target("avx2,fma,f16c"))) float dot_q6k_avx2(const BlockQ6_K* w, const BlockQ8_0* x, int nsb) {
  const __m256i m4 = _mm256_set1_epi8(0xF), m2 = _mm256_set1_epi8(3), one = _mm256_set1_epi8(1);
  __m256 acc = _mm256_setzero_ps();
  for (int i = 0; i < nsb; ++i) {
    const float d = f16_to_f32(w[i].d);
    for (int half = 0; half < 2; ++half) {
      const __m256i l0 = _mm256_loadu_si256((const __m256i*)(w[i].ql + 64 * half));
      const __m256i l1 = _mm256_loadu_si256((const __m256i*)(w[i].ql + 64 * half + 32));
      const __m256i h = _mm256_loadu_si256((const __m256i*)(w[i].qh + 32 * half));
      const int8_t* sc = w[i].scales + 8 * half;
      // the four 32-value parts of this half: low nibbles of ql[0..31], of ql[32..63], then the high nibbles
      const __m256i nib[4] = {_mm256_and_si256(l0, m4), _mm256_and_si256(l1, m4),
                              _mm256_and_si256(_mm256_srli_epi16(l0, 4), m4), _mm256_and_si256(_mm256_srli_epi16(l1, 4), m4)};
      const __m256i top[4] = {_mm256_and_si256(h, m2), _mm256_and_si256(_mm256_srli_epi16(h, 2), m2),
                              _mm256_and_si256(_mm256_srli_epi16(h, 4), m2), _mm256_and_si256(_mm256_srli_epi16(h, 6), m2)};
      for (int part = 0; part < 4; ++part) {
        const BlockQ8_0& xb = x[i * 8 + half * 4 + part];
        const __m256i xv = _mm256_loadu_si256((const __m256i*)xb.qs);
        const __m256i qu = _mm256_or_si256(nib[part], _mm256_slli_epi16(top[part], 4));     // 0 .. 63
        // sum(qu * x) - 32 sum(x) per group of 16, then the group's scale
        const __m256i sums = _mm256_sub_epi32(mul_sum_i32(qu, xv), _mm256_slli_epi32(mul_sum_i32(one, xv), 5));
        const float dd = f16_to_f32(xb.d) * d;
        const float sa = dd * (float)sc[2 * part], sb = dd * (float)sc[2 * part + 1];
        acc = _mm256_fmadd_ps(_mm256_cvtepi32_ps(sums), _mm256_set_ps(sb, sb, sb, sb, sa, sa, sa, sa), acc);
      }
    }
  }
  return hsum_f32(acc);
}
#endif

typedef float (*DotQ4kFn)(const BlockQ4_K*, const BlockQ8_0*, int);
typedef float (*DotQ6kFn)(const BlockQ6_K*, const BlockQ8_0*, int);
DotQ4kFn pick_dot_q4k(int level) {
#if defined(__x86_64__)
  if (level >= 2) return dot_q4k_avx2;
#endif
  (void)level;
  return dot_q4k_scalar;
}
DotQ6kFn pick_dot_q6k(int level) {
#if defined(__x86_64__)
  if (level >= 2) return dot_q6k_avx2;
#endif
  (void)level;
  return dot_q6k_scalar;
}

float dot_f32(const float* a, const float* b, int n) {
  float s0 = 0, s1 = 0, s2 = 0, s3 = 0;
  int i = 0;
  for (; i + 4 <= n; i += 4) {
    s0 += a[i] * b[i]; s1 += a[i + 1] * b[i + 1]; s2 += a[i + 2] * b[i + 2]; s3 += a[i + 3] * b[i + 3];
  }
  for (; i < n; ++i) s0 += a[i] * b[i];
  return (s0 + s1) + (s2 + s3);
}

// ------------------------------------------------------------------------------ worker pool
// Chunk indices are handed out from one 64-bit word that also carries the task's generation, so a
// worker that wakes late (after its task has finished and the next one has been posted) can never
// take a chunk of the new task with the old task's function: its compare-exchange fails on the
// generation.  The caller leaves run() only when every chunk is done and no worker is still
// inside the task.
class Pool {
 public:
  explicit Pool(int n) : n_(n < 1 ? 1 : n) {
    for (int i = 1; i < n_; ++i) threads_.emplace_back([this] { loop(); });
  }
  ~Pool() {
    {
      std::lock_guard<std::mutex> g(mu_);
      stop_ = true;
      gen_.fetch_add(1, std::memory_order_release);
    }
    cv_.notify_all();
    for (auto& t : threads_) t.join();
  }
  int size() const { return n_; }

  // fn(chunk) for chunk in [0, chunks); returns when all are done.
  template <class F>
  void run(int chunks, F&& fn) {
    if (chunks <= 0) return;
    if (n_ == 1 || chunks == 1) {
      for (int c = 0; c < chunks; ++c) fn(c);
      return;
    }
    struct Task {
      F* fn;
      static void call(void* self, int c) { (*static_cast<Task*>(self)->fn)(c); }
    } task{&fn};
    unsigned g;
    {
      std::lock_guard<std::mutex> lk(mu_);
      call_ = &Task::call;
      arg_ = &task;
      chunks_ = chunks;
      done_.store(0, std::memory_order_relaxed);
      g = gen_.load(std::memory_order_relaxed) + 1;
      ticket_.store((uint64_t)g << 32, std::memory_order_relaxed);
      gen_.store(g, std::memory_order_release);
    }
    cv_.notify_all();
    work(g, &Task::call, &task, chunks);
    while (done_.load(std::memory_order_acquire) < chunks) cpu_relax();
    while (inside_.load(std::memory_order_acquire) > 0) cpu_relax();
  }

 private:
  static void cpu_relax() {
#if defined(__x86_64__)
    _mm_pause();
#endif
  }
  void work(unsigned g, void (*call)(void*, int), void* arg, int chunks) {
    for (;;) {
      uint64_t t = ticket_.load(std::memory_order_acquire);
      if ((unsigned)(t >> 32) != g) return;          // another task owns the counter now
      const int c = (int)(t & 0xffffffffu);
      if (c >= chunks) return;
      if (!ticket_.compare_exchange_weak(t, t + 1, std::memory_order_acq_rel)) continue;
      call(arg, c);
      done_.fetch_add(1, std::memory_order_release);
    }
  }
  void loop() {
    unsigned seen = 0;
    for (;;) {
      int spins = 0;
      while (gen_.load(std::memory_order_acquire) == seen) {
        if (++spins < 512) {
          cpu_relax();
          continue;
        }
        std::unique_lock<std::mutex> l(mu_);
        cv_.wait(l, [&] { return gen_.load(std::memory_order_acquire) != seen; });
      }
      void (*call)(void*, int);
      void* arg;
      int chunks;
      {
        std::lock_guard<std::mutex> lk(mu_);
        if (stop_) return;
        seen = gen_.load(std::memory_order_acquire);
        call = call_;
        arg = arg_;
        chunks = chunks_;
        inside_.fetch_add(1, std::memory_order_acq_rel);
      }
      work(seen, call, arg, chunks);
      inside_.fetch_sub(1, std::memory_order_acq_rel);
    }
  }

  int n_;
  std::vector<std::thread> threads_;
  std::mutex mu_;
  std::condition_variable cv_;
  std::atomic<unsigned> gen_{0};
  std::atomic<uint64_t> ticket_{0};
  std::atomic<int> done_{0}, inside_{0};
  void (*call_)(void*, int) = nullptr;
  void* arg_ = nullptr;
  int chunks_ = 0;
  bool stop_ = false;
};

// ------------------------------------------------------------------------------ model
enum Role { R_ATTN_NORM, R_Q, R_K, R_V, R_O, R_Q_NORM, R_K_NORM, R_FFN_NORM, R_GATE, R_UP, R_DOWN, R_BQ, R_BK, R_BV,
            R_COUNT };
enum GlobalRole { G_EMBED = 100, G_OUT_NORM = 101, G_LM_HEAD = 102 };

struct Tensor {
  const void* data = nullptr;
  int type = -1;
};

struct Layer {
  Tensor t[R_COUNT];
  std::vector<float> attn_norm, ffn_norm, q_norm, k_norm, bq, bk, bv;   // small vectors cached as f32
  std::vector<BlockQ8_0> k, v;   // [cap, n_kv, hd/32]
};

struct Model {
  LkCpuConfig c;
  std::vector<Layer> layers;
  Tensor embed, out_norm_t, lm_head;
  std::vector<float> out_norm, inv_freq;
  int cap = 0;     // positions the KV cache holds room for
  int level = 0;
  DotFn dot = dot_q8_scalar;
  Pool* pool = nullptr;
  // arena
  std::vector<float> x, h, q, k, v, attn, proj, gate, up, scores, rowbuf;
  std::vector<BlockQ8_0> hq, attnq, actq, qq;
};

void to_f32(const Tensor& t, int n, std::vector<float>& out) {
  out.resize(n);
  if (!t.data) {
    out.clear();
    return;
  }
  if (t.type == T_F32) memcpy(out.data(), t.data, sizeof(float) * n);
  else if (t.type == T_F16) for (int i = 0; i < n; ++i) out[i] = f16_to_f32(((const uint16_t*)t.data)[i]);
  else if (t.type == T_BF16) for (int i = 0; i < n; ++i) out[i] = bf16_to_f32(((const uint16_t*)t.data)[i]);
  else dequant_any(t.type, t.data, out.data(), n);
}

size_t row_bytes(int type, int K) {
  const TypeInfo ti = type_info(type);
  return (size_t)K / ti.block_values * ti.block_bytes;
}

void dequant_row(const Tensor& t, long long row, int K, float* dst) {
  const uint8_t* p = (const uint8_t*)t.data + row * row_bytes(t.type, K);
  if (t.type == T_F32) memcpy(dst, p, sizeof(float) * K);
  else if (t.type == T_F16) for (int i = 0; i < K; ++i) dst[i] = f16_to_f32(((const uint16_t*)p)[i]);
  else if (t.type == T_BF16) for (int i = 0; i < K; ++i) dst[i] = bf16_to_f32(((const uint16_t*)p)[i]);
  else dequant_any(t.type, p, dst, K);
}

// out[N] = W[N, K] x.  Q8_0 weights take the integer dot with the quantised activation `xq`;
// anything else is expanded a row at a time and multiplied in f32 with `xf`.
void gemv(Model& m, const Tensor& w, int N, int K, const BlockQ8_0* xq, const float* xf, float* out) {
  const int nb = K / 32;
  const int chunk = 32;
  const int chunks = (N + chunk - 1) / chunk;
  if (w.type == T_Q8_0) {
    const BlockQ8_0* W = (const BlockQ8_0*)w.data;
    DotFn dot = m.dot;
    m.pool->run(chunks, [&](int c) {
      const int r1 = (c + 1) * chunk < N ? (c + 1) * chunk : N;
      for (int r = c * chunk; r < r1; ++r) out[r] = dot(W + (size_t)r * nb, xq, nb);
    });
    return;
  }
  if ((w.type == T_Q4_K || w.type == T_Q6_K) && K % 256 == 0 && xq) {
    const int nsb = K / 256;
    if (w.type == T_Q4_K) {
      const BlockQ4_K* W = (const BlockQ4_K*)w.data;
      DotQ4kFn dot = pick_dot_q4k(m.level);
      m.pool->run(chunks, [&](int c) {
        const int r1 = (c + 1) * chunk < N ? (c + 1) * chunk : N;
        for (int r = c * chunk; r < r1; ++r) out[r] = dot(W + (size_t)r * nsb, xq, nsb);
      });
    } else {
      const BlockQ6_K* W = (const BlockQ6_K*)w.data;
      DotQ6kFn dot = pick_dot_q6k(m.level);
      m.pool->run(chunks, [&](int c) {
        const int r1 = (c + 1) * chunk < N ? (c + 1) * chunk : N;
        for (int r = c * chunk; r < r1; ++r) out[r] = dot(W + (size_t)r * nsb, xq, nsb);
      });
    }
    return;
  }
  m.pool->run(chunks, [&](int c) {
    std::vector<float> row(K);
    const int r1 = (c + 1) * chunk < N ? (c + 1) * chunk : N;
    for (int r = c * chunk; r < r1; ++r) {
      dequant_row(w, r, K, row.data());
      out[r] = dot_f32(row.data(), xf, K);
    }
  });
}

void rmsnorm(const float* x, const float* w, int n, float eps, float* out) {
  double ss = 0;
  for (int i = 0; i < n; ++i) ss += (double)x[i] * x[i];
  const float r = 1.0f / sqrtf((float)(ss / n) + eps);
  for (int i = 0; i < n; ++i) out[i] = x[i] * r * w[i];
}

void rope(float* v, int hd, int rope_dim, int pairing, int pos, const float* inv_freq) {
  const int half = rope_dim / 2;
  for (int i = 0; i < half; ++i) {
    const float a = (float)pos * inv_freq[i];
    const float c = cosf(a), s = sinf(a);
    const int i0 = pairing == 0 ? 2 * i : i;
    const int i1 = pairing == 0 ? 2 * i + 1 : i + half;
    const float x0 = v[i0], x1 = v[i1];
    v[i0] = x0 * c - x1 * s;
    v[i1] = x0 * s + x1 * c;
  }
  (void)hd;
}

void ensure_cap(Model& m, int need) {
  if (need <= m.cap) return;
  int cap = m.cap ? m.cap : 256;
  while (cap < need) cap *= 2;
  const size_t per_pos = (size_t)m.c.n_kv * (m.c.head_dim / 32);
  for (auto& L : m.layers) {
    L.k.resize(per_pos * cap);
    L.v.resize(per_pos * cap);
  }
  m.scores.resize((size_t)m.c.n_q * cap);
  m.cap = cap;
}

int decode_one(Model& m, int token, int pos, float* logits) {
  const LkCpuConfig& c = m.c;
  const int H = c.hidden, hd = c.head_dim, nq = c.n_q, nkv = c.n_kv, I = c.intermediate;
  const int G = nq / nkv, hb = hd / 32;
  if (token < 0 || token >= c.vocab || pos < 0) return -1;
  ensure_cap(m, pos + 1);
  dequant_row(m.embed, token, H, m.x.data());
  const float scale = 1.0f / sqrtf((float)hd);
  for (int il = 0; il < c.n_layers; ++il) {
    Layer& L = m.layers[il];
    rmsnorm(m.x.data(), L.attn_norm.data(), H, c.rms_eps, m.h.data());
    quant_q8_0(m.h.data(), m.hq.data(), H);
    gemv(m, L.t[R_Q], nq * hd, H, m.hq.data(), m.h.data(), m.q.data());
    gemv(m, L.t[R_K], nkv * hd, H, m.hq.data(), m.h.data(), m.k.data());
    gemv(m, L.t[R_V], nkv * hd, H, m.hq.data(), m.h.data(), m.v.data());
    if (!L.bq.empty()) for (int i = 0; i < nq * hd; ++i) m.q[i] += L.bq[i];
    if (!L.bk.empty()) for (int i = 0; i < nkv * hd; ++i) m.k[i] += L.bk[i];
    if (!L.bv.empty()) for (int i = 0; i < nkv * hd; ++i) m.v[i] += L.bv[i];
    for (int h = 0; h < nq; ++h) {
      float* qh = m.q.data() + h * hd;
      if (!L.q_norm.empty()) rmsnorm(qh, L.q_norm.data(), hd, c.rms_eps, qh);
      rope(qh, hd, c.rope_dim, c.rope_pairing, pos, m.inv_freq.data());
    }
    const size_t per_pos = (size_t)nkv * hb;
    for (int h = 0; h < nkv; ++h) {
      float* kh = m.k.data() + h * hd;
      if (!L.k_norm.empty()) rmsnorm(kh, L.k_norm.data(), hd, c.rms_eps, kh);
      rope(kh, hd, c.rope_dim, c.rope_pairing, pos, m.inv_freq.data());
      quant_q8_0(kh, &L.k[per_pos * pos + (size_t)h * hb], hd);
      quant_q8_0(m.v.data() + h * hd, &L.v[per_pos * pos + (size_t)h * hb], hd);
    }
    quant_q8_0(m.q.data(), m.qq.data(), nq * hd);
    const int n_keys = pos + 1;
    DotFn dot = m.dot;
    m.pool->run(nq, [&](int h) {
      const int kvh = h / G;
      float* sc = m.scores.data() + (size_t)h * m.cap;
      const BlockQ8_0* qv = m.qq.data() + (size_t)h * hb;
      float mx = -INFINITY;
      for (int t = 0; t < n_keys; ++t) {
        sc[t] = dot(&L.k[per_pos * t + (size_t)kvh * hb], qv, hb) * scale;
        mx = sc[t] > mx ? sc[t] : mx;
      }
      float sum = 0.f;
      for (int t = 0; t < n_keys; ++t) {
        sc[t] = expf(sc[t] - mx);
        sum += sc[t];
      }
      const float inv = 1.0f / sum;
      float* o = m.attn.data() + (size_t)h * hd;
      for (int i = 0; i < hd; ++i) o[i] = 0.f;
      for (int t = 0; t < n_keys; ++t) {
        const BlockQ8_0* vb = &L.v[per_pos * t + (size_t)kvh * hb];
        const float p = sc[t] * inv;
        for (int b = 0; b < hb; ++b) {
          const float pd = p * f16_to_f32(vb[b].d);
          for (int i = 0; i < 32; ++i) o[b * 32 + i] += pd * (float)vb[b].qs[i];
        }
      }
    });
    quant_q8_0(m.attn.data(), m.attnq.data(), nq * hd);
    gemv(m, L.t[R_O], H, nq * hd, m.attnq.data(), m.attn.data(), m.proj.data());
    for (int i = 0; i < H; ++i) m.x[i] += m.proj[i];
    rmsnorm(m.x.data(), L.ffn_norm.data(), H, c.rms_eps, m.h.data());
    quant_q8_0(m.h.data(), m.hq.data(), H);
    gemv(m, L.t[R_GATE], I, H, m.hq.data(), m.h.data(), m.gate.data());
    gemv(m, L.t[R_UP], I, H, m.hq.data(), m.h.data(), m.up.data());
    for (int i = 0; i < I; ++i) {
      const float g = m.gate[i];
      m.gate[i] = g / (1.0f + expf(-g)) * m.up[i];
    }
    quant_q8_0(m.gate.data(), m.actq.data(), I);
    gemv(m, L.t[R_DOWN], H, I, m.actq.data(), m.gate.data(), m.proj.data());
    for (int i = 0; i < H; ++i) m.x[i] += m.proj[i];
  }
  if (logits) {
    rmsnorm(m.x.data(), m.out_norm.data(), H, c.rms_eps, m.h.data());
    quant_q8_0(m.h.data(), m.hq.data(), H);
    gemv(m, m.lm_head.data ? m.lm_head : m.embed, c.vocab, H, m.hq.data(), m.h.data(), logits);
  }
  return 0;
}

}  // namespace

// ------------------------------------------------------------------------------ C API
LKH_API void* lkcpu_create(const LkCpuConfig* cfg, int threads, int max_level) {
  if (!cfg || cfg->head_dim % 32 || cfg->hidden % 32 || cfg->intermediate % 32 || cfg->n_q % cfg->n_kv) return nullptr;
  Model* m = new Model();
  m->c = *cfg;
  m->layers.resize(cfg->n_layers);
  int level = lkc_cpu_level();
  if (max_level >= 0 && max_level < level) level = max_level;
  m->level = level;
  m->dot = pick_dot(level);
  if (threads <= 0) {
    threads = (int)std::thread::hardware_concurrency();
    if (threads > 1) threads = threads / 2 > 0 ? threads : 1;
  }
  m->pool = new Pool(threads);
  const int H = cfg->hidden, hd = cfg->head_dim, I = cfg->intermediate;
  m->x.resize(H); m->h.resize(H); m->proj.resize(H);
  m->q.resize((size_t)cfg->n_q * hd); m->k.resize((size_t)cfg->n_kv * hd); m->v.resize((size_t)cfg->n_kv * hd);
  m->attn.resize((size_t)cfg->n_q * hd);
  m->gate.resize(I); m->up.resize(I);
  m->hq.resize(H / 32); m->attnq.resize((size_t)cfg->n_q * hd / 32); m->actq.resize(I / 32);
  m->qq.resize((size_t)cfg->n_q * hd / 32);
  const int rd = cfg->rope_dim > 0 ? cfg->rope_dim : hd;
  m->c.rope_dim = rd;
  m->inv_freq.resize(rd / 2);
  for (int i = 0; i < rd / 2; ++i) m->inv_freq[i] = 1.0f / powf(cfg->rope_theta, (float)(2 * i) / (float)rd);
  return m;
}

LKH_API void lkcpu_free(void* h) {
  Model* m = (Model*)h;
  if (!m) return;
  delete m->pool;
  delete m;
}

LKH_API int lkcpu_set_inv_freq(void* h, const float* inv_freq, int n) {
  Model* m = (Model*)h;
  if (!m || n != (int)m->inv_freq.size()) return -1;
  memcpy(m->inv_freq.data(), inv_freq, sizeof(float) * n);
  return 0;
}

// layer < 0: role is one of 100 (token embedding), 101 (output norm), 102 (lm head).
// The data must stay mapped while the model lives (it usually points into the GGUF mapping).
LKH_API int lkcpu_set_tensor(void* h, int layer, int role, const void* data, int type) {
  Model* m = (Model*)h;
  if (!m || !data) return -1;
  const LkCpuConfig& c = m->c;
  Tensor t{data, type};
  if (layer < 0) {
    if (role == G_EMBED) m->embed = t;
    else if (role == G_LM_HEAD) m->lm_head = t;
    else if (role == G_OUT_NORM) to_f32(t, c.hidden, m->out_norm);
    else return -1;
    return 0;
  }
  if (layer >= c.n_layers || role < 0 || role >= R_COUNT) return -1;
  Layer& L = m->layers[layer];
  L.t[role] = t;
  const int hd = c.head_dim;
  switch (role) {
    case R_ATTN_NORM: to_f32(t, c.hidden, L.attn_norm); break;
    case R_FFN_NORM: to_f32(t, c.hidden, L.ffn_norm); break;
    case R_Q_NORM: to_f32(t, hd, L.q_norm); break;
    case R_K_NORM: to_f32(t, hd, L.k_norm); break;
    case R_BQ: to_f32(t, c.n_q * hd, L.bq); break;
    case R_BK: to_f32(t, c.n_kv * hd, L.bk); break;
    case R_BV: to_f32(t, c.n_kv * hd, L.bv); break;
    default: break;
  }
  return 0;
}

LKH_API int lkcpu_ready(void* h) {
  Model* m = (Model*)h;
  if (!m || !m->embed.data || m->out_norm.empty()) return 0;
  for (auto& L : m->layers) {
    if (L.attn_norm.empty() || L.ffn_norm.empty()) return 0;
    for (int r : {R_Q, R_K, R_V, R_O, R_GATE, R_UP, R_DOWN})
      if (!L.t[r].data) return 0;
  }
  return 1;
}

// Feeds `token` at position `pos` (positions must arrive in order from 0, or from a position
// already in the cache to overwrite from there).  `logits` may be null while a prompt is fed.
LKH_API int lkcpu_decode(void* h, int token, int pos, float* logits) {
  Model* m = (Model*)h;
  if (!m || !lkcpu_ready(h)) return -2;
  return decode_one(*m, token, pos, logits);
}

LKH_API int lkcpu_level(void* h) { return h ? ((Model*)h)->level : -1; }
LKH_API int lkcpu_threads(void* h) { return h ? ((Model*)h)->pool->size() : -1; }

// ------------------------------------------------------------------------------ experts on the host
// (token, expert) pairs of a mixture layer computed on the host cores, over expert matrices held in host memory
// in the DEVICE plane layouts (ops/quant.py: codes plane + scale-record plane), so the same pinned buffers serve
// the copy into a GPU slot and this path.  Used for experts that are not resident on the GPU at decode size:
// computing a pair here reads the expert's bytes once from host memory instead of sending them over the bus
// (reference: src/inference/moe_cuda_cpu/, the expert tier's "compute misses beside the card").
//   fmt 0  bf16 rows
//   fmt 1  Q8_0: int8 codes, one f16 scale per 32 values
//   fmt 2  Q6_K: int8 codes (centred), per 256 values f16 d + sixteen int8 scales (one per 16 values)
//   fmt 3  Q4_K: nibbles (value k in byte k / 2, the even one low), per 256 values f16 d, f16 dmin, eight
//          6-bit scales and eight 6-bit minima as bytes
//   fmt 4  MXFP4: E2M1 nibbles in the same order, one E8M0 exponent byte per 32 values (the scale plane's row
//          pitch is passed: it is padded for the block-scaled MMA)
// Activations are quantised per 32 values (d = amax / 127); for Q4_K their codes are stored even values first,
// then odd ones, per group, to line up with the nibbles.
namespace {

struct PlaneAct {
  std::vector<int8_t> q;      // [K] (per group of 32: natural order, or evens then odds)
  std::vector<float> d, sum;  // [K / 32]: scale, and d * sum of the codes
};

void quant_plane_act(const float* x, int K, bool split, PlaneAct& a) {
  const int ng = K / 32;
  a.q.resize(K);
  a.d.resize(ng);
  a.sum.resize(ng);
  for (int g = 0; g < ng; ++g) {
    float amax = 0.f;
    for (int j = 0; j < 32; ++j) amax = std::max(amax, fabsf(x[g * 32 + j]));
    const float d = amax / 127.f, id = d ? 1.f / d : 0.f;
    int s = 0;
    for (int j = 0; j < 32; ++j) {
      const int q = (int)lroundf(x[g * 32 + j] * id);
      s += q;
      const int at = split ? ((j & 1) ? 16 + (j >> 1) : (j >> 1)) : j;
      a.q[g * 32 + at] = (int8_t)q;
    }
    a.d[g] = d;
    a.sum[g] = d * (float)s;
  }
}

#if defined(__x86_64__)
__attribute__((target("avx2"))) static inline int32_t dot32_s8(const int8_t* w, const int8_t* x) {
  const __m256i a = _mm256_loadu_si256((const __m256i*)w), c = _mm256_loadu_si256((const __m256i*)x);
  const __m256i p16 = _mm256_maddubs_epi16(_mm256_sign_epi8(a, a), _mm256_sign_epi8(c, a));
  return hsum_i32(_mm256_madd_epi16(p16, _mm256_set1_epi16(1)));
}
__attribute__((target("avx2"))) static inline void dot16x2_s8(const int8_t* w, const int8_t* x, int32_t* lo, int32_t* hi) {
  const __m256i a = _mm256_loadu_si256((const __m256i*)w), c = _mm256_loadu_si256((const __m256i*)x);
  const __m256i p32 = _mm256_madd_epi16(_mm256_maddubs_epi16(_mm256_sign_epi8(a, a), _mm256_sign_epi8(c, a)),
                                        _mm256_set1_epi16(1));
  __m128i l = _mm256_castsi256_si128(p32), h = _mm256_extracti128_si256(p32, 1);
  l = _mm_add_epi32(l, _mm_shuffle_epi32(l, 0x4E));
  l = _mm_add_epi32(l, _mm_shuffle_epi32(l, 0xB1));
  h = _mm_add_epi32(h, _mm_shuffle_epi32(h, 0x4E));
  h = _mm_add_epi32(h, _mm_shuffle_epi32(h, 0xB1));
  *lo = _mm_cvtsi128_si32(l);
  *hi = _mm_cvtsi128_si32(h);
}
// sixteen bytes of nibbles against evens-then-odds activation codes
__attribute__((target("avx2"))) static inline int32_t dot32_nib(const uint8_t* w, const int8_t* x) {
  const __m128i b = _mm_loadu_si128((const __m128i*)w);
  const __m128i m4 = _mm_set1_epi8(0xF);
  const __m256i q = _mm256_set_m128i(_mm_and_si128(_mm_srli_epi16(b, 4), m4), _mm_and_si128(b, m4));
  const __m256i c = _mm256_loadu_si256((const __m256i*)x);
  return hsum_i32(_mm256_madd_epi16(_mm256_maddubs_epi16(q, c), _mm256_set1_epi16(1)));
}
#endif

// one row of a plane matrix times a quantised (or, for bf16, float) activation
float plane_row_dot(int fmt, const uint8_t* codes, const uint8_t* scales, int K, const PlaneAct& a, const float* xf, int level) {
  const int ng = K / 32;
  float acc = 0.f;
  (void)level;
  if (fmt == 0) {
    const uint16_t* w = (const uint16_t*)codes;
    for (int k = 0; k < K; ++k) acc += bf16_to_f32(w[k]) * xf[k];
    return acc;
  }
  if (fmt == 1) {
    const uint16_t* dw = (const uint16_t*)scales;
    for (int g = 0; g < ng; ++g) {
      int32_t s = 0;
#if defined(__x86_64__)
      if (level >= 2) s = dot32_s8((const int8_t*)codes + g * 32, a.q.data() + g * 32);
      else
#endif
        for (int j = 0; j < 32; ++j) s += (int32_t)((const int8_t*)codes)[g * 32 + j] * a.q[g * 32 + j];
      acc += f16_to_f32(dw[g]) * a.d[g] * (float)s;
    }
    return acc;
  }
  if (fmt == 2) {
    for (int g = 0; g < ng; ++g) {
      const uint8_t* rec = scales + (g >> 3) * 18;
      const float d = f16_to_f32(*(const uint16_t*)rec);
      const int8_t* sc = (const int8_t*)rec + 2 + (g & 7) * 2;
      int32_t lo = 0, hi = 0;
#if defined(__x86_64__)
      if (level >= 2) dot16x2_s8((const int8_t*)codes + g * 32, a.q.data() + g * 32, &lo, &hi);
      else
#endif
        for (int j = 0; j < 16; ++j) {
          lo += (int32_t)((const int8_t*)codes)[g * 32 + j] * a.q[g * 32 + j];
          hi += (int32_t)((const int8_t*)codes)[g * 32 + 16 + j] * a.q[g * 32 + 16 + j];
        }
      acc += d * a.d[g] * ((float)sc[0] * (float)lo + (float)sc[1] * (float)hi);
    }
    return acc;
  }
  if (fmt == 4) {
    // codes are E2M1 values times two (the LUT of formats.h); 2^(e - 127) / 2 puts them back
    for (int g = 0; g < ng; ++g) {
      int32_t s = 0;
      for (int b = 0; b < 16; ++b) {
        s += (int32_t)kMxfp4Lut[codes[g * 16 + b] & 0xF] * a.q[g * 32 + b];
        s += (int32_t)kMxfp4Lut[codes[g * 16 + b] >> 4] * a.q[g * 32 + 16 + b];
      }
      acc += 0.5f * e8m0_to_f32(scales[g]) * a.d[g] * (float)s;
    }
    return acc;
  }
  // fmt 3
  for (int g = 0; g < ng; ++g) {
    const uint8_t* rec = scales + (g >> 3) * 20;
    const int j = g & 7;
    const float d = f16_to_f32(*(const uint16_t*)rec) * (float)rec[4 + j];
    const float mn = f16_to_f32(*(const uint16_t*)(rec + 2)) * (float)rec[12 + j];
    int32_t s = 0;
#if defined(__x86_64__)
    if (level >= 2) s = dot32_nib(codes + g * 16, a.q.data() + g * 32);
    else
#endif
      for (int b = 0; b < 16; ++b) {
        s += (int32_t)(codes[g * 16 + b] & 0xF) * a.q[g * 32 + b];
        s += (int32_t)(codes[g * 16 + b] >> 4) * a.q[g * 32 + 16 + b];
      }
    acc += d * a.d[g] * (float)s - mn * a.sum[g];
  }
  return acc;
}

size_t plane_code_bytes(int fmt, int K) { return fmt == 0 ? (size_t)K * 2 : fmt >= 3 ? (size_t)K / 2 : (size_t)K; }
size_t plane_scale_bytes(int fmt, int K) {
  return fmt == 0 ? 0 : fmt == 1 ? (size_t)K / 16 : fmt == 2 ? (size_t)K / 256 * 18 : fmt == 4 ? (size_t)K / 32
                                                                                               : (size_t)K / 256 * 20;
}

}  // namespace

// out[t] += w * down_e(glu(gate_up_e(x[t]))) for every pair (t = pair_tok[p], e = pair_expert[p], w = pair_w[p]).
// gate_up stacks 2I rows per expert (gate rows, then up rows) of width H, down stacks H rows of width I; planes are
// contiguous.  x and out are f32 [T, H]; biases f32 [E, 2I] / [E, H] or null.  Returns 0, or -1 for a bad argument.
LKH_API int lkcpu_moe_pairs(int fmt_gu, const void* gu_codes, const void* gu_scales, int fmt_dn, const void* dn_codes,
                            const void* dn_scales, const float* gu_bias, const float* dn_bias, int H, int I,
                            const float* x, const int* pair_tok, const int* pair_expert, const float* pair_w, int n_pairs,
                            int glu_mode, float alpha, float limit, float* out, int threads, int max_level,
                            long long gu_scale_pitch, long long dn_scale_pitch) {
  if (n_pairs <= 0) return 0;
  if (!gu_codes || !dn_codes || !x || !out || !pair_tok || !pair_expert || !pair_w || (H % 32) || (I % 32)) return -1;
  if (fmt_gu < 0 || fmt_gu > 4 || fmt_dn < 0 || fmt_dn > 4) return -1;
  if (((fmt_gu == 2 || fmt_gu == 3) && (H % 256)) || ((fmt_dn == 2 || fmt_dn == 3) && (I % 256))) return -1;
  if ((fmt_gu && !gu_scales) || (fmt_dn && !dn_scales)) return -1;
  int level = lkc_cpu_level();
  if (max_level >= 0 && max_level < level) level = max_level;
  Pool pool(threads);
  const size_t gcb = plane_code_bytes(fmt_gu, H), gsb = gu_scale_pitch > 0 ? (size_t)gu_scale_pitch : plane_scale_bytes(fmt_gu, H);
  const size_t dcb = plane_code_bytes(fmt_dn, I), dsb = dn_scale_pitch > 0 ? (size_t)dn_scale_pitch : plane_scale_bytes(fmt_dn, I);
  std::vector<float> gu((size_t)n_pairs * 2 * I), y((size_t)n_pairs * H);
  std::vector<PlaneAct> ax(n_pairs), aa(n_pairs);
  std::vector<std::vector<float>> act(n_pairs);
  for (int p = 0; p < n_pairs; ++p) quant_plane_act(x + (size_t)pair_tok[p] * H, H, fmt_gu >= 3, ax[p]);
  const int chunk = 64;
  const int gch = (2 * I + chunk - 1) / chunk;
  pool.run(n_pairs * gch, [&](int task) {
    const int p = task / gch, c = task % gch;
    const size_t e = (size_t)pair_expert[p];
    const uint8_t* cw = (const uint8_t*)gu_codes + e * 2 * I * gcb;
    const uint8_t* sw = gu_scales ? (const uint8_t*)gu_scales + e * 2 * I * gsb : nullptr;
    const float* xf = x + (size_t)pair_tok[p] * H;
    const int r1 = std::min(2 * I, (c + 1) * chunk);
    for (int r = c * chunk; r < r1; ++r)
      gu[(size_t)p * 2 * I + r] = plane_row_dot(fmt_gu, cw + r * gcb, sw ? sw + r * gsb : nullptr, H, ax[p], xf, level) +
                                  (gu_bias ? gu_bias[e * 2 * I + r] : 0.f);
  });
  for (int p = 0; p < n_pairs; ++p) {
    act[p].resize(I);
    const float* g = gu.data() + (size_t)p * 2 * I;
    for (int i = 0; i < I; ++i) {
      if (glu_mode == 0) {
        act[p][i] = g[i] / (1.f + expf(-g[i])) * g[I + i];
      } else {
        const float gg = std::min(g[i], limit), uu = std::min(std::max(g[I + i], -limit), limit);
        act[p][i] = gg / (1.f + expf(-alpha * gg)) * (1.f + uu);
      }
    }
    quant_plane_act(act[p].data(), I, fmt_dn >= 3, aa[p]);
  }
  const int dch = (H + chunk - 1) / chunk;
  pool.run(n_pairs * dch, [&](int task) {
    const int p = task / dch, c = task % dch;
    const size_t e = (size_t)pair_expert[p];
    const uint8_t* cw = (const uint8_t*)dn_codes + e * H * dcb;
    const uint8_t* sw = dn_scales ? (const uint8_t*)dn_scales + e * H * dsb : nullptr;
    const int r1 = std::min(H, (c + 1) * chunk);
    for (int r = c * chunk; r < r1; ++r)
      y[(size_t)p * H + r] = plane_row_dot(fmt_dn, cw + r * dcb, sw ? sw + r * dsb : nullptr, I, aa[p], act[p].data(), level) +
                             (dn_bias ? dn_bias[e * H + r] : 0.f);
  });
  for (int p = 0; p < n_pairs; ++p) {          // in pair order: the sum of a token's pairs does not depend on threads
    float* o = out + (size_t)pair_tok[p] * H;
    const float w = pair_w[p];
    for (int r = 0; r < H; ++r) o[r] += w * y[(size_t)p * H + r];
  }
  return 0;
}

// Test hooks: the dot at a forced SIMD level, and a pooled GEMV.
LKH_API float lkcpu_dot_q8_0(const void* x, const void* y, int nblocks, int level) {
  int have = lkc_cpu_level();
  if (level > have) level = have;
  return pick_dot(level)((const BlockQ8_0*)x, (const BlockQ8_0*)y, nblocks);
}

// The same for any stored row type (`type`: the file's type code; Q8_0, Q4_K and Q6_K take integer dots with
// the Q8_0-quantised activation, the rest a row dequantiser and an f32 dot).
LKH_API int lkcpu_gemv_any(int type, const void* w, const float* x, float* out, int N, int K, int threads, int level) {
  if (K % 32) return -1;
  Model m;
  int have = lkc_cpu_level();
  m.level = level > have ? have : level;
  m.dot = pick_dot(m.level);
  Pool pool(threads);
  m.pool = &pool;
  std::vector<BlockQ8_0> xq(K / 32);
  quant_q8_0(x, xq.data(), K);
  Tensor t{w, type};
  gemv(m, t, N, K, xq.data(), x, out);
  m.pool = nullptr;
  return 0;
}

LKH_API int lkcpu_gemv_q8_0(const void* w, const float* x, float* out, int N, int K, int threads, int level) {
  if (K % 32) return -1;
  Model m;
  int have = lkc_cpu_level();
  m.dot = pick_dot(level > have ? have : level);
  Pool pool(threads);
  m.pool = &pool;
  std::vector<BlockQ8_0> xq(K / 32);
  quant_q8_0(x, xq.data(), K);
  Tensor t{w, T_Q8_0};
  gemv(m, t, N, K, xq.data(), x, out);
  m.pool = nullptr;
  return 0;
}
