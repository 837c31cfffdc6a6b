// Range checks of the debug build (-DWX_CHECK). In a release build every macro below compiles to nothing.
//
// compute-sanitizer style checking without a tool: with -DWX_CHECK the kernels test the indices, tensor-map
// coordinates, bulk-copy alignments and barrier phases they are about to use. A violation is *recorded* (first
// offending site and its two values, plus a count) and the access is skipped; nothing traps, asserts or spins, so the
// context stays usable and the host reads the record afterwards (binding `check_report`). The record lives in one
// device array per translation unit (no relocatable device code is needed); WX_CHK_DEFINE_READER gives each unit a
// host function that copies it out and clears it.
//
// Site ids: 1xxx ptx helpers (TMA / bulk copies / mbarrier / TMEM), 2xxx gemm, 3xxx attention, 4xxx kernels,
// 5xxx index, 6xxx comm, 7xxx decode.
#pragma once
#include <cuda_runtime.h>

#ifdef WX_CHECK
namespace wx {
namespace chk {
static __device__ unsigned long long g_record[4];  // [0] first site, [1] violations, [2], [3] values at the first site
__device__ __forceinline__ bool fail(int site, long long v0, long long v1) {
  if (atomicCAS(&g_record[0], 0ull, static_cast<unsigned long long>(site)) == 0ull) {
    g_record[2] = static_cast<unsigned long long>(v0);
    g_record[3] = static_cast<unsigned long long>(v1);
  }
  atomicAdd(&g_record[1], 1ull);
  return false;
}
}  // namespace chk
}  // namespace wx
// true when `cond` holds; otherwise records (site, v0, v1) and yields false so that the caller skips the access
#define WX_CHK(cond, site, v0, v1) ((cond) ? true : wx::chk::fail((site), static_cast<long long>(v0), static_cast<long long>(v1)))
#define WX_CHK_DEFINE_READER(name)                                                                      \
  int name(long long* out4, int clear) {                                                                \
    unsigned long long h[4] = {0, 0, 0, 0};                                                             \
    cudaError_t e = cudaMemcpyFromSymbol(h, wx::chk::g_record, sizeof(h));                              \
    if (e == cudaSuccess && clear && h[1] != 0) {                                                       \
      const unsigned long long z[4] = {0, 0, 0, 0};                                                     \
      e = cudaMemcpyToSymbol(wx::chk::g_record, z, sizeof(z));                                          \
    }                                                                                                   \
    for (int i = 0; i < 4; ++i) out4[i] = static_cast<long long>(h[i]);                                 \
    return static_cast<int>(e);                                                                         \
  }
#define WX_CHECKED_BUILD 1
#else
#define WX_CHK(cond, site, v0, v1) (true)
#define WX_CHK_DEFINE_READER(name)             \
  int name(long long* out4, int) {             \
    out4[0] = out4[1] = out4[2] = out4[3] = 0; \
    return 0;                                  \
  }
#define WX_CHECKED_BUILD 0
#endif
