// Host-side helpers shared by the launchers: error codes, TMA tensor-map creation through
// the driver entry point (no link-time dependency on libcuda), launch counting.
#pragma once
#include <stdlib.h>
#include <string.h>
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define LK_API extern "C" __attribute__((visibility("default")))

// Return codes of every launcher: 0 = launched, negative = refused before launch,
// positive = CUDA runtime error code.
enum { LKH_OK = 0, LKH_BAD_ARG = -1, LKH_NO_DRIVER = -2, LKH_TMAP_FAIL = -3, LKH_TOO_LARGE = -4 };

namespace lkh {

// number of kernel launches issued by this library since load (read by the bench to
// report how many of its own kernels ran inside the timed region)
extern unsigned long long g_launches;
inline void count_launch(int n = 1) { g_launches += (unsigned long long)n; }

inline PFN_cuTensorMapEncodeTiled get_encode_fn() {
  static PFN_cuTensorMapEncodeTiled fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled>(p);
  }
  return fn;
}

// 2-D row-major tensor [rows, cols] of `esize`-byte elements, row pitch `ld_bytes`.
// Box = box_rows x box_cols with the 128-byte swizzle (box_cols * esize must be 128).
// Out-of-range elements read as zero, so ragged edges in any dimension need no special case.
inline int make_tmap_2d(CUtensorMap* tm, const void* base, CUtensorMapDataType dt, int esize, uint64_t rows,
                        uint64_t cols, uint64_t ld_bytes, uint32_t box_rows, uint32_t box_cols) {
  PFN_cuTensorMapEncodeTiled enc = get_encode_fn();
  if (!enc) return LKH_NO_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld_bytes & 15) || box_rows > 256 || box_cols * esize != 128)
    return LKH_BAD_ARG;
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstr[1] = {ld_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(tm, dt, 2, const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? LKH_OK : LKH_TMAP_FAIL;
}

// 2-D row-major byte tensor [rows, row_bytes] read in boxes of box_rows x box_bytes WITHOUT swizzle
// (shared-memory image = the box's rows back to back); box_bytes a multiple of 16.
inline int make_tmap_2d_plain(CUtensorMap* tm, const void* base, uint64_t rows, uint64_t row_bytes, uint64_t ld_bytes,
                              uint32_t box_rows, uint32_t box_bytes) {
  PFN_cuTensorMapEncodeTiled enc = get_encode_fn();
  if (!enc) return LKH_NO_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld_bytes & 15) || box_rows > 256 || (box_bytes & 15) || box_bytes > 256)
    return LKH_BAD_ARG;
  cuuint64_t gdim[2] = {row_bytes, rows};
  cuuint64_t gstr[1] = {ld_bytes};
  cuuint32_t box[2] = {box_bytes, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), gdim, gstr, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? LKH_OK : LKH_TMAP_FAIL;
}

// 3-D variant: [d2, rows, cols] with byte pitches ld1 (row) and ld2 (outer).
inline int make_tmap_3d(CUtensorMap* tm, const void* base, CUtensorMapDataType dt, int esize, uint64_t d2,
                        uint64_t rows, uint64_t cols, uint64_t ld1, uint64_t ld2, uint32_t box_rows,
                        uint32_t box_cols) {
  PFN_cuTensorMapEncodeTiled enc = get_encode_fn();
  if (!enc) return LKH_NO_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld1 & 15) || (ld2 & 15) || box_rows > 256 ||
      box_cols * esize != 128)
    return LKH_BAD_ARG;
  cuuint64_t gdim[3] = {cols, rows, d2};
  cuuint64_t gstr[2] = {ld1, ld2};
  cuuint32_t box[3] = {box_cols, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(tm, dt, 3, const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? LKH_OK : LKH_TMAP_FAIL;
}

inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? LKH_OK : static_cast<int>(e);
}

// Programmatic dependent launch for the kernels of the decode step: the kernel may be scheduled
// while its predecessor in the stream is still running, so its launch latency and its prologue
// (barrier set-up, TMEM allocation, descriptor prefetch) overlap the predecessor's tail.  Every
// kernel launched this way executes `griddepcontrol.wait` (lk::pdl_wait) in every CTA before it
// touches global memory and before any early return; that wait ends when the predecessor has
// completed and its writes are visible, so the chain stays ordered.  LOKEN_PDL=0 turns it off.
inline bool pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("LOKEN_PDL");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on == 1;
}
template <typename... KArgs, typename... Args>
inline void launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

}  // namespace lkh
