// Split-KV decode attention with its workspace in the library's own device image: the entry
// point for callers that may not allocate (contract in loken_noalloc.h).  Nothing here calls an
// allocating routine; the only set-up is one address look-up per CUDA context.
#include "loken_noalloc.h"
#include "host_common.h"
#include <mutex>

namespace {

// counters first (they are the part that must start at zero), partial results after them
constexpr size_t kCounterBytes = sizeof(int) * LK_DECODE_STATIC_COUNTERS;
constexpr size_t kScratchBytes = kCounterBytes + sizeof(float) * (size_t)LK_DECODE_STATIC_WS_FLOATS;
static_assert(kCounterBytes % 256 == 0, "the float region keeps the array's alignment");

static __device__ __align__(256) unsigned char g_decode_scratch[kScratchBytes];

// The array's address belongs to the CUDA context it was looked up in, not to the device ordinal:
// a plug-in may be called from several contexts on one device, and a context may be destroyed and
// made again (cudaDeviceReset).  The look-up is therefore remembered per context handle; a
// handle that was never seen (or that the driver hands out again after a reset, whose address is
// then re-validated by the cheap pointer-attribute query below) is resolved afresh.
constexpr int kMaxContexts = 64;
struct CtxEntry {
  CUcontext ctx;
  void* ptr;
};
CtxEntry g_ctx_table[kMaxContexts];
int g_ctx_count = 0;
std::mutex g_ctx_mutex;

typedef CUresult (*CtxGetCurrentFn)(CUcontext*);
CtxGetCurrentFn ctx_get_current_fn() {
  static CtxGetCurrentFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuCtxGetCurrent", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<CtxGetCurrentFn>(p);
  }
  return fn;
}

// Address of the array in the context that is current on the calling thread.
int scratch_for_current_context(void** out) {
  // make sure the runtime has a context current on this thread (no-op once it has)
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  CUcontext ctx = nullptr;
  CtxGetCurrentFn get = ctx_get_current_fn();
  if (get && get(&ctx) != CUDA_SUCCESS) ctx = nullptr;
  std::lock_guard<std::mutex> lock(g_ctx_mutex);
  if (ctx) {
    for (int i = 0; i < g_ctx_count; ++i) {
      if (g_ctx_table[i].ctx == ctx) {
        // a destroyed context's handle can come back for a new context: the remembered address
        // must still be device memory of the current context, else it is looked up again
        cudaPointerAttributes at;
        if (cudaPointerGetAttributes(&at, g_ctx_table[i].ptr) == cudaSuccess && at.type == cudaMemoryTypeDevice &&
            at.device == dev) {
          *out = g_ctx_table[i].ptr;
          return LKH_OK;
        }
        (void)cudaGetLastError();
        g_ctx_table[i] = g_ctx_table[--g_ctx_count];
        break;
      }
    }
  }
  void* ptr = nullptr;
  e = cudaGetSymbolAddress((void**)&ptr, g_decode_scratch);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (!ptr || (reinterpret_cast<uintptr_t>(ptr) & 255)) return LKH_BAD_ARG;
  if (ctx && g_ctx_count < kMaxContexts) g_ctx_table[g_ctx_count++] = CtxEntry{ctx, ptr};
  *out = ptr;       // no context handle or a full table: the address is simply looked up every call
  return LKH_OK;
}

}  // namespace

LK_API void lk_attn_decode_static_limits(long long* ws_floats, int* counters) {
  if (ws_floats) *ws_floats = LK_DECODE_STATIC_WS_FLOATS;
  if (counters) *counters = LK_DECODE_STATIC_COUNTERS;
}

LK_API int lk_attn_decode_static(const LkDecodeArgs* a, void* stream) {
  if (!a) return LKH_BAD_ARG;
  if (a->rows <= 0) return LKH_OK;
  if (a->n_kv <= 0 || a->n_q <= 0 || a->n_q % a->n_kv) return LKH_BAD_ARG;
  const int nsplit = a->nsplit < 1 ? 1 : a->nsplit;
  if (nsplit == 1) {
    // one block per (row, kv head) writes its result itself: no partial results, no counters, so
    // no limit applies and the array is not touched
    LkDecodeArgs b = *a;
    b.counters = nullptr;
    b.n_counters = 0;
    b.ws = nullptr;
    b.ws_floats = 0;
    return lk_attn_decode(&b, stream);
  }
  const long long need_ws = lk_attn_decode_ws_floats(a->rows, a->n_q, a->n_kv, a->hd, nsplit);
  const long long need_ctr = (long long)a->rows * a->n_kv;
  if (need_ws > LK_DECODE_STATIC_WS_FLOATS || need_ctr > LK_DECODE_STATIC_COUNTERS) {
    fprintf(stderr,
            "lk_attn_decode_static: rows=%d n_q=%d n_kv=%d hd=%d nsplit=%d needs %lld workspace floats and %lld "
            "counters; the fixed array holds %d and %d\n",
            a->rows, a->n_q, a->n_kv, a->hd, nsplit, need_ws, need_ctr, (int)LK_DECODE_STATIC_WS_FLOATS,
            (int)LK_DECODE_STATIC_COUNTERS);
    return LKH_TOO_LARGE;
  }
  void* base = nullptr;
  const int rc = scratch_for_current_context(&base);
  if (rc != LKH_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  // the arrival counters of this call's (row, kv head) pairs start at zero
  cudaError_t e = cudaMemsetAsync(base, 0, sizeof(int) * (size_t)need_ctr, st);
  if (e != cudaSuccess) return static_cast<int>(e);
  LkDecodeArgs b = *a;
  b.counters = reinterpret_cast<int*>(base);
  b.n_counters = LK_DECODE_STATIC_COUNTERS;
  b.ws = reinterpret_cast<float*>(static_cast<unsigned char*>(base) + kCounterBytes);
  b.ws_floats = LK_DECODE_STATIC_WS_FLOATS;
  return lk_attn_decode(&b, stream);
}
