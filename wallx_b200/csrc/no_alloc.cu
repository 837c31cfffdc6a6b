// Allocation-free variant of the column-sum kernel (see no_alloc.h for who needs it and why).
//
// The fp32 accumulator that the regular path gets from the allocator is a file-scope device array
// here. Host code cannot use the array's name as a pointer: on the host that name is only a
// stand-in for the symbol, and a kernel handed it would fault, or would quietly read and write
// the wrong memory on systems where the GPU can reach host memory. The device address is
// therefore resolved with cudaGetSymbolAddress, once per device, and that pointer is what the
// kernels receive.
#include "no_alloc.h"

#include <cuda_bf16.h>
#include <mutex>

namespace {

static __device__ __align__(256) float g_noalloc_scratch[WX_NOALLOC_MAX_COLS];

constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {nullptr};
std::mutex g_setup_mutex;

// Device address of the scratch array on the current device (resolved on first use).
float* scratch_for_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch) != cudaSuccess) return nullptr;
    g_scratch_ptr[dev] = p;
  }
  return g_scratch_ptr[dev];
}

__global__ void noalloc_clear_kernel(float* __restrict__ acc, int cols) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < cols) acc[i] = 0.f;
}

// Each block sums a slice of rows for 256 columns (two per thread) and adds it into `acc`.
__global__ void noalloc_column_sum_kernel(const __nv_bfloat16* __restrict__ x, long ld, float* __restrict__ acc,
                                          int rows, int cols, int rows_per_block) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (c >= cols) return;
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(rows, r0 + rows_per_block);
  const bool pair = (c + 1 < cols) && ((ld & 1) == 0);
  float s0 = 0.f, s1 = 0.f;
  for (int r = r0; r < r1; ++r) {
    const __nv_bfloat16* p = x + static_cast<long>(r) * ld + c;
    if (pair) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
      s0 += f.x;
      s1 += f.y;
    } else {
      s0 += __bfloat162float(p[0]);
      if (c + 1 < cols) s1 += __bfloat162float(p[1]);
    }
  }
  atomicAdd(&acc[c], s0);
  if (c + 1 < cols) atomicAdd(&acc[c + 1], s1);
}

__global__ void noalloc_store_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ out, int cols) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < cols) out[i] = __float2bfloat16(acc[i]);
}

}  // namespace

extern "C" int wx_column_sum_bf16_noalloc(const void* x, long ld, void* out, int rows, int cols, cudaStream_t stream) {
  if (x == nullptr || out == nullptr || rows < 0 || cols < 0 || ld < cols) return WX_NOALLOC_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(x) & 3) != 0) return WX_NOALLOC_ERR_BAD_ARG;
  if (cols > WX_NOALLOC_MAX_COLS) return WX_NOALLOC_ERR_TOO_WIDE;
  if (cols == 0) return WX_NOALLOC_OK;
  float* acc = scratch_for_current_device();
  if (acc == nullptr) return WX_NOALLOC_ERR_SETUP;
  // The array still holds the previous call's sums: clear the part this call accumulates into.
  noalloc_clear_kernel<<<(cols + 255) / 256, 256, 0, stream>>>(acc, cols);
  if (rows > 0) {
    int ysplit = (rows + 255) / 256;
    if (ysplit > 256) ysplit = 256;
    const int rows_per_block = (rows + ysplit - 1) / ysplit;
    const int pairs = (cols + 1) / 2;
    dim3 grid((pairs + 127) / 128, ysplit);
    noalloc_column_sum_kernel<<<grid, 128, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), ld, acc, rows, cols,
                                                        rows_per_block);
  }
  noalloc_store_kernel<<<(cols + 255) / 256, 256, 0, stream>>>(acc, reinterpret_cast<__nv_bfloat16*>(out), cols);
  return static_cast<int>(cudaGetLastError());
}

extern "C" const char* wx_noalloc_strerror(int code) {
  switch (code) {
    case WX_NOALLOC_OK: return "ok";
    case WX_NOALLOC_ERR_BAD_ARG: return "bad argument: null pointer, negative size, ld < cols or misaligned input";
    case WX_NOALLOC_ERR_TOO_WIDE: return "cols exceeds WX_NOALLOC_MAX_COLS (65536): the built-in scratch array is too small";
    case WX_NOALLOC_ERR_SETUP: return "could not resolve the device address of the built-in scratch array on this device";
    default: return code > 0 ? cudaGetErrorString(static_cast<cudaError_t>(code)) : "unknown error";
  }
}
