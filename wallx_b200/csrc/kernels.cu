// Bandwidth- and latency-bound kernels: RMSNorm (+ fused token-type permutation), rotary on the
// packed q|k|v buffer, SwiGLU backward, routing plan for the dual-expert FFN, row permutation,
// column sums, cross entropy over a logits block, grad-norm and fused AdamW on flat buffers.
// All of them use 16-byte accesses and take an explicit stream.
//
// Reference parity: csrc/permute.cu (row map + gather/scatter), csrc/rope.cu (mRoPE fwd/bwd), the
// ATen chains behind Qwen2RMSNorm (modeling_qwen2_5_vl.py:122-139), SiLU*mul, CrossEntropyLoss
// and torch.optim.AdamW (qwen_vl_act_trainer.py:577-581).
#include "kernels.h"
#include "check.cuh"
#include "devinfo.h"
#include "launch.h"

#include <cuda_bf16.h>
#include <math.h>

namespace wx {

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; `red` is a shared float[32]. Every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = (lane < nw) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = (lane < nw) ? red[lane] : -INFINITY;
  t = warp_max(t);
  return t;
}

struct alignas(16) BF8 {
  __nv_bfloat162 v[4];
};
__device__ __forceinline__ void unpack8(const BF8& b, float* f) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(b.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ BF8 pack8(const float* f) {
  BF8 b;
#pragma unroll
  for (int i = 0; i < 4; ++i) b.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return b;
}
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16(x)); }

constexpr int NORM_THREADS = 256;
constexpr int NORM_MAX_CHUNKS = 4;  // C <= 256 * 8 * 4 = 8192

// ------------------------------------------------------------------------------ RMSNorm forward
__global__ void __launch_bounds__(NORM_THREADS)
rms_norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                    __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out, const int* __restrict__ dest, int T,
                    int C, float eps) {
  __shared__ float red[32];
  const int nchunk = C >> 3;
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const BF8* xr = reinterpret_cast<const BF8*>(x + static_cast<size_t>(row) * C);
    float v[NORM_MAX_CHUNKS][8];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < NORM_MAX_CHUNKS; ++c) {
      const int i = threadIdx.x + c * NORM_THREADS;
      if (i < nchunk) {
        unpack8(xr[i], v[c]);
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += v[c][e] * v[c][e];
      }
    }
    ss = block_sum(ss, red);
    const float rstd = rsqrtf(ss / static_cast<float>(C) + eps);
    if (threadIdx.x == 0) rstd_out[row] = rstd;
    const int orow = dest ? dest[row] : row;
    BF8* yr = reinterpret_cast<BF8*>(y + static_cast<size_t>(orow) * C);
    const BF8* wr = reinterpret_cast<const BF8*>(w);
#pragma unroll
    for (int c = 0; c < NORM_MAX_CHUNKS; ++c) {
      const int i = threadIdx.x + c * NORM_THREADS;
      if (i < nchunk) {
        float wf[8], o[8];
        unpack8(wr[i], wf);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = wf[e] * bf16_round(v[c][e] * rstd);
        yr[i] = pack8(o);
      }
    }
  }
}

// ------------------------------------------------------------------------------ RMSNorm backward
// dx = rstd * (g - xhat * mean(g * xhat)), g = dy * w, xhat = x * rstd; dw partials per block.
__global__ void __launch_bounds__(NORM_THREADS)
rms_norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                    const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                    const int* __restrict__ dest, __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_partial, int T,
                    int C, const __nv_bfloat16* __restrict__ add) {
  __shared__ float red[32];
  const int nchunk = C >> 3;
  float dwacc[NORM_MAX_CHUNKS][8];
#pragma unroll
  for (int c = 0; c < NORM_MAX_CHUNKS; ++c)
#pragma unroll
    for (int e = 0; e < 8; ++e) dwacc[c][e] = 0.f;
  const BF8* wr = reinterpret_cast<const BF8*>(w);
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const int grow = dest ? dest[row] : row;
    const BF8* xr = reinterpret_cast<const BF8*>(x + static_cast<size_t>(row) * C);
    const BF8* gr = reinterpret_cast<const BF8*>(dy + static_cast<size_t>(grow) * C);
    const float rstd = rstd_in[row];
    float xh[NORM_MAX_CHUNKS][8], g[NORM_MAX_CHUNKS][8];
    float dot = 0.f;
#pragma unroll
    for (int c = 0; c < NORM_MAX_CHUNKS; ++c) {
      const int i = threadIdx.x + c * NORM_THREADS;
      if (i < nchunk) {
        float xf[8], df[8], wf[8];
        unpack8(xr[i], xf);
        unpack8(gr[i], df);
        unpack8(wr[i], wf);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          xh[c][e] = xf[e] * rstd;
          g[c][e] = df[e] * wf[e];
          dot += g[c][e] * xh[c][e];
          dwacc[c][e] += df[e] * bf16_round(xh[c][e]);
        }
      }
    }
    dot = block_sum(dot, red) / static_cast<float>(C);
    BF8* dxr = reinterpret_cast<BF8*>(dx + static_cast<size_t>(row) * C);
#pragma unroll
    for (int c = 0; c < NORM_MAX_CHUNKS; ++c) {
      const int i = threadIdx.x + c * NORM_THREADS;
      if (i < nchunk) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = rstd * (g[c][e] - xh[c][e] * dot);
        if (add != nullptr) {  // + the gradient of the residual path, with the rounding of a separate bf16 add
          float af[8];
          unpack8(reinterpret_cast<const BF8*>(add + static_cast<size_t>(row) * C)[i], af);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = bf16_round(o[e]) + af[e];
        }
        dxr[i] = pack8(o);
      }
    }
  }
  float* dp = dw_partial + static_cast<size_t>(blockIdx.x) * C;
#pragma unroll
  for (int c = 0; c < NORM_MAX_CHUNKS; ++c) {
    const int i = threadIdx.x + c * NORM_THREADS;
    if (i < nchunk) {
#pragma unroll
      for (int e = 0; e < 8; ++e) dp[i * 8 + e] = dwacc[c][e];
    }
  }
}

// ------------------------------------------------------------------------------ RMSNorm, one warp per row
// For C = 256 * CH <= 2048 a warp owns a whole row: CH 16-byte loads per lane are in flight at
// once and the reduction is shuffles only (no block barrier per row). Eight rows per block.
// EARLY_W (few rows: the kernel is one chain of latencies) requests the weight chunks together with the row instead of
// after the reduction; with many rows the extra registers would cost occupancy, so the streaming case keeps them late.
template <int CH, bool EARLY_W>
__global__ void __launch_bounds__(256)
rms_norm_fwd_warp_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                         __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out, const int* __restrict__ dest,
                         int T, float eps) {
  constexpr int C = CH * 256;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const BF8* wr = reinterpret_cast<const BF8*>(w);
  pdl_wait();
  pdl_launch_dependents();
  for (int row = blockIdx.x * 8 + warp; row < T; row += gridDim.x * 8) {
    const BF8* xr = reinterpret_cast<const BF8*>(x + static_cast<size_t>(row) * C);
    BF8 raw[CH], wraw[EARLY_W ? CH : 1];
#pragma unroll
    for (int c = 0; c < CH; ++c) raw[c] = xr[lane + 32 * c];
    if (EARLY_W) {
#pragma unroll
      for (int c = 0; c < CH; ++c) wraw[c] = wr[lane + 32 * c];
    }
    float v[CH][8];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      unpack8(raw[c], v[c]);
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[c][e] * v[c][e];
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / static_cast<float>(C) + eps);
    if (lane == 0) rstd_out[row] = rstd;
    const int orow = dest ? dest[row] : row;
    BF8* yr = reinterpret_cast<BF8*>(y + static_cast<size_t>(orow) * C);
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      float wf[8], o[8];
      unpack8(EARLY_W ? wraw[c] : wr[lane + 32 * c], wf);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = wf[e] * bf16_round(v[c][e] * rstd);
      yr[lane + 32 * c] = pack8(o);
    }
  }
}

template <int CH>
__global__ void __launch_bounds__(256)
rms_norm_bwd_warp_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                         const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                         const int* __restrict__ dest, __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_partial,
                         int T, const __nv_bfloat16* __restrict__ add) {
  constexpr int C = CH * 256;
  __shared__ float dws[C];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < C; i += 256) dws[i] = 0.f;
  __syncthreads();
  float dwacc[CH][8];
#pragma unroll
  for (int c = 0; c < CH; ++c)
#pragma unroll
    for (int e = 0; e < 8; ++e) dwacc[c][e] = 0.f;
  const BF8* wr = reinterpret_cast<const BF8*>(w);
  for (int row = blockIdx.x * 8 + warp; row < T; row += gridDim.x * 8) {
    const int grow = dest ? dest[row] : row;
    const BF8* xr = reinterpret_cast<const BF8*>(x + static_cast<size_t>(row) * C);
    const BF8* gr = reinterpret_cast<const BF8*>(dy + static_cast<size_t>(grow) * C);
    const float rstd = rstd_in[row];
    BF8 xraw[CH], graw[CH], araw[CH];
    // all loads of the row are issued together (the residual-path gradient too: loading it after the reduction
    // would put a second memory round trip on every row's critical path)
    const BF8* ar = add != nullptr ? reinterpret_cast<const BF8*>(add + static_cast<size_t>(row) * C) : nullptr;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      xraw[c] = xr[lane + 32 * c];
      graw[c] = gr[lane + 32 * c];
      if (ar != nullptr) araw[c] = ar[lane + 32 * c];
    }
    float dot = 0.f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      float xf[8], df[8], wf[8];
      unpack8(xraw[c], xf);
      unpack8(graw[c], df);
      unpack8(wr[lane + 32 * c], wf);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float xh = xf[e] * rstd;
        dot += df[e] * wf[e] * xh;
        dwacc[c][e] += df[e] * bf16_round(xh);
      }
    }
    dot = warp_sum(dot) / static_cast<float>(C);
    BF8* dxr = reinterpret_cast<BF8*>(dx + static_cast<size_t>(row) * C);
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      float xf[8], df[8], wf[8], o[8];
      unpack8(xraw[c], xf);
      unpack8(graw[c], df);
      unpack8(wr[lane + 32 * c], wf);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = rstd * (df[e] * wf[e] - xf[e] * rstd * dot);
      if (ar != nullptr) {  // + the gradient of the residual path, with the rounding of a separate bf16 add
        float af[8];
        unpack8(araw[c], af);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = bf16_round(o[e]) + af[e];
      }
      dxr[lane + 32 * c] = pack8(o);
    }
  }
  // warps add their sums one after the other, so the result does not depend on timing
  for (int wv = 0; wv < 8; ++wv) {
    if (warp == wv) {
#pragma unroll
      for (int c = 0; c < CH; ++c)
#pragma unroll
        for (int e = 0; e < 8; ++e) dws[(lane + 32 * c) * 8 + e] += dwacc[c][e];
    }
    __syncthreads();
  }
  float* dp = dw_partial + static_cast<size_t>(blockIdx.x) * C;
  for (int i = threadIdx.x; i < C; i += 256) dp[i] = dws[i];
}

__global__ void reduce_partials_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out, int nblk,
                                       int C) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s = 0.f;
  for (int b = 0; b < nblk; ++b) s += partial[static_cast<size_t>(b) * C + c];
  out[c] = __float2bfloat16(s);
}

// ------------------------------------------------------------------------------ SwiGLU backward
// gu is [R, ld_gu] with 32-column blocks [16 gate | 16 up]; dh is [R, ld_dh]. One thread handles 8
// gate and the matching 8 up channels (three 16-byte loads, two 16-byte stores); neighbouring
// threads take neighbouring 16-byte chunks, so every 32-byte sector is used whole.
__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dh, const __nv_bfloat16* __restrict__ gu,
                  __nv_bfloat16* __restrict__ dgu, int R, int nblk, long ld_dh, long ld_gu) {
  const long per_row = static_cast<long>(nblk) * 2;
  const long total = static_cast<long>(R) * per_row;
  for (long idx = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(idx / per_row);
    const int rem = static_cast<int>(idx - static_cast<long>(r) * per_row);
    const int b = rem >> 1, h = rem & 1;
    const __nv_bfloat16* grow = gu + r * ld_gu + b * 32 + h * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(*reinterpret_cast<const BF8*>(grow), g);
    unpack8(*reinterpret_cast<const BF8*>(grow + 16), u);
    unpack8(*reinterpret_cast<const BF8*>(dh + r * ld_dh + b * 16 + h * 8), d);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float sg = 1.f / (1.f + __expf(-g[e]));
      du[e] = d[e] * g[e] * sg;
      dg[e] = d[e] * u[e] * (sg * (1.f + g[e] * (1.f - sg)));
    }
    __nv_bfloat16* orow = dgu + r * ld_gu + b * 32 + h * 8;
    *reinterpret_cast<BF8*>(orow) = pack8(dg);
    *reinterpret_cast<BF8*>(orow + 16) = pack8(du);
  }
}

// ------------------------------------------------------------------------------ rotary on q|k|v
// One thread owns 8 channels of the first half of the head dimension (and their partners in the
// second half) of one token and walks over all rotated heads with them, so the fp32 cos/sin
// values are loaded once per token instead of once per head; the v columns (heads >= n_rot) are
// copied by the same threads. `inverse` applies the transposed rotation (the backward pass).
__global__ void __launch_bounds__(256)
rope_qk_kernel(const __nv_bfloat16* in, __nv_bfloat16* out, const float* __restrict__ cos_t,
               const float* __restrict__ sin_t, int T, int W, int n_rot, int D, int inverse, int copy_rest) {
  const int half = D >> 1;
  const int tpr = half >> 3;  // threads per token
  const long idx = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long>(T) * tpr) return;
  const int t = static_cast<int>(idx / tpr);
  const int d0 = static_cast<int>(idx - static_cast<long>(t) * tpr) * 8;
  const __nv_bfloat16* row = in + static_cast<size_t>(t) * W;
  __nv_bfloat16* orow = out + static_cast<size_t>(t) * W;
  const float* cs = cos_t + static_cast<size_t>(t) * D;
  const float* sn = sin_t + static_cast<size_t>(t) * D;
  float c1[8], s1[8], c2[8], s2[8];  // 16-byte loads: d0 is a multiple of 8 floats, rows are 16-byte aligned
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    *reinterpret_cast<float4*>(c1 + 4 * q) = *reinterpret_cast<const float4*>(cs + d0 + 4 * q);
    *reinterpret_cast<float4*>(s1 + 4 * q) = *reinterpret_cast<const float4*>(sn + d0 + 4 * q);
    *reinterpret_cast<float4*>(c2 + 4 * q) = *reinterpret_cast<const float4*>(cs + half + d0 + 4 * q);
    *reinterpret_cast<float4*>(s2 + 4 * q) = *reinterpret_cast<const float4*>(sn + half + d0 + 4 * q);
  }
#pragma unroll 2
  for (int h = 0; h < n_rot; ++h) {
    float a[8], b[8], oa[8], ob[8];
    unpack8(*reinterpret_cast<const BF8*>(row + h * D + d0), a);
    unpack8(*reinterpret_cast<const BF8*>(row + h * D + half + d0), b);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      if (!inverse) {
        oa[e] = a[e] * c1[e] - b[e] * s1[e];
        ob[e] = b[e] * c2[e] + a[e] * s2[e];
      } else {
        oa[e] = a[e] * c1[e] + b[e] * s2[e];
        ob[e] = b[e] * c2[e] - a[e] * s1[e];
      }
    }
    *reinterpret_cast<BF8*>(orow + h * D + d0) = pack8(oa);
    *reinterpret_cast<BF8*>(orow + h * D + half + d0) = pack8(ob);
  }
  // pass-through columns, 16 bytes at a time, spread over the token's threads (nothing to do in place)
  if (!copy_rest) return;
  const int base = n_rot * D;
  for (int off = base + d0; off < W; off += tpr * 8)
    *reinterpret_cast<BF8*>(orow + off) = *reinterpret_cast<const BF8*>(row + off);
}

// Variant for few tokens (decoding, the denoise loop): one thread per (token, head, 8-channel chunk), so that
// a handful of tokens still spreads over many SMs; it reloads cos/sin per head.
__global__ void rope_qk_chunk_kernel(const __nv_bfloat16* in, __nv_bfloat16* out, const float* __restrict__ cos_t,
                                     const float* __restrict__ sin_t, int T, int W, int n_rot, int D, int inverse,
                                     int copy_rest) {
  const int half = D >> 1;
  const int chunks_per_head = half >> 3;
  const int rot_chunks = n_rot * chunks_per_head;
  const int copy_chunks = copy_rest ? (W - n_rot * D) >> 3 : 0;
  const int per_row = rot_chunks + copy_chunks;
  const long idx = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long>(T) * per_row) return;
  const int t = static_cast<int>(idx / per_row);
  const int c = static_cast<int>(idx - static_cast<long>(t) * per_row);
  const __nv_bfloat16* row = in + static_cast<size_t>(t) * W;
  __nv_bfloat16* orow = out + static_cast<size_t>(t) * W;
  if (c >= rot_chunks) {
    const int off = n_rot * D + (c - rot_chunks) * 8;
    *reinterpret_cast<BF8*>(orow + off) = *reinterpret_cast<const BF8*>(row + off);
    return;
  }
  const int h = c / chunks_per_head;
  const int d0 = (c - h * chunks_per_head) * 8;
  float a[8], b[8], oa[8], ob[8];
  unpack8(*reinterpret_cast<const BF8*>(row + h * D + d0), a);
  unpack8(*reinterpret_cast<const BF8*>(row + h * D + half + d0), b);
  const float* cs = cos_t + static_cast<size_t>(t) * D;
  const float* sn = sin_t + static_cast<size_t>(t) * D;
  float c1[8], s1[8], c2[8], s2[8];  // 16-byte loads: d0 is a multiple of 8 floats, rows are 16-byte aligned
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    *reinterpret_cast<float4*>(c1 + 4 * q) = *reinterpret_cast<const float4*>(cs + d0 + 4 * q);
    *reinterpret_cast<float4*>(s1 + 4 * q) = *reinterpret_cast<const float4*>(sn + d0 + 4 * q);
    *reinterpret_cast<float4*>(c2 + 4 * q) = *reinterpret_cast<const float4*>(cs + half + d0 + 4 * q);
    *reinterpret_cast<float4*>(s2 + 4 * q) = *reinterpret_cast<const float4*>(sn + half + d0 + 4 * q);
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    if (!inverse) {
      oa[e] = a[e] * c1[e] - b[e] * s1[e];
      ob[e] = b[e] * c2[e] + a[e] * s2[e];
    } else {
      oa[e] = a[e] * c1[e] + b[e] * s2[e];
      ob[e] = b[e] * c2[e] - a[e] * s1[e];
    }
  }
  *reinterpret_cast<BF8*>(orow + h * D + d0) = pack8(oa);
  *reinterpret_cast<BF8*>(orow + h * D + half + d0) = pack8(ob);
}

// ------------------------------------------------------------------------------ routing plan
// Single block: stable grouping of T tokens by expert id (E <= 8) with 128-row aligned segments.
constexpr int ROUTE_THREADS = 1024;
constexpr int ROUTE_MAX_E = 8;
__global__ void __launch_bounds__(ROUTE_THREADS)
route_plan_kernel(const int* __restrict__ types, int T, int E, int rows, int* __restrict__ dest,
                  int* __restrict__ seg, int* __restrict__ segk, int* __restrict__ inv) {
  __shared__ int counts[ROUTE_MAX_E];
  __shared__ int starts[ROUTE_MAX_E];
  __shared__ int warp_cnt[ROUTE_MAX_E][32];
  __shared__ int running[ROUTE_MAX_E];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x < ROUTE_MAX_E) counts[threadIdx.x] = 0;
  for (int i = threadIdx.x; i < rows; i += ROUTE_THREADS) inv[i] = -1;
  __syncthreads();
  // pass 1: counts
  int local[ROUTE_MAX_E];
#pragma unroll
  for (int e = 0; e < ROUTE_MAX_E; ++e) local[e] = 0;
  for (int i = threadIdx.x; i < T; i += ROUTE_THREADS) {
    const int tt = types[i];
#pragma unroll
    for (int e = 0; e < ROUTE_MAX_E; ++e) local[e] += (tt == e);
  }
#pragma unroll
  for (int e = 0; e < ROUTE_MAX_E; ++e) {
    int v = local[e];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0 && v && e < E) atomicAdd(&counts[e], v);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int s = 0;
    for (int e = 0; e < E; ++e) {
      const int c = counts[e];
      const int p = (c + 127) / 128 * 128;
      starts[e] = s;
      running[e] = s;
      seg[e * 4 + 0] = s;
      seg[e * 4 + 1] = c;
      seg[e * 4 + 2] = -1;
      seg[e * 4 + 3] = -1;
      segk[e * 4 + 0] = -1;
      segk[e * 4 + 1] = -1;
      segk[e * 4 + 2] = s;
      segk[e * 4 + 3] = p;
      s += p;
    }
  }
  __syncthreads();
  // pass 2: stable ranks, chunk by chunk
  for (int base = 0; base < T; base += ROUTE_THREADS) {
    const int i = base + threadIdx.x;
    const int tt = (i < T) ? types[i] : -1;
    if (i < T) (void)WX_CHK(tt >= 0 && tt < E, 4002, tt, E);  // a token type outside the expert range is dropped
    int my_rank = 0;
    for (int e = 0; e < E; ++e) {
      const unsigned bal = __ballot_sync(0xffffffffu, tt == e);
      if (tt == e) my_rank = __popc(bal & ((1u << lane) - 1u));
      if (lane == 0) warp_cnt[e][warp] = __popc(bal);
    }
    __syncthreads();
    if (tt >= 0 && tt < E) {
      int off = running[tt];
      for (int w2 = 0; w2 < warp; ++w2) off += warp_cnt[tt][w2];
      const int d = off + my_rank;
      dest[i] = d;
      if (WX_CHK(d >= 0 && d < rows, 4001, d, rows)) inv[d] = i;
    }
    __syncthreads();
    if (threadIdx.x < E) {
      int s = 0;
      for (int w2 = 0; w2 < 32; ++w2) s += warp_cnt[threadIdx.x][w2];
      running[threadIdx.x] += s;
    }
    __syncthreads();
  }
}

// out[dest[t], :] = x[t, :]; out is zero-filled by the caller.
__global__ void permute_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ dest,
                                    __nv_bfloat16* __restrict__ out, int T, int C, int out_rows) {
  const int nchunk = C >> 3;
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    if (!WX_CHK(dest[row] >= 0 && (out_rows <= 0 || dest[row] < out_rows) && (C & 7) == 0, 4003, dest[row], out_rows)) continue;
    const BF8* src = reinterpret_cast<const BF8*>(x + static_cast<size_t>(row) * C);
    BF8* dst = reinterpret_cast<BF8*>(out + static_cast<size_t>(dest[row]) * C);
    for (int i = threadIdx.x; i < nchunk; i += blockDim.x) dst[i] = src[i];
  }
}

// out[t, :] = x[idx[t], :]
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ idx,
                                   __nv_bfloat16* __restrict__ out, int T, int C, int src_rows) {
  const int nchunk = C >> 3;
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    if (!WX_CHK(idx[row] >= 0 && (src_rows <= 0 || idx[row] < src_rows) && (C & 7) == 0, 4004, idx[row], src_rows)) continue;
    const BF8* src = reinterpret_cast<const BF8*>(x + static_cast<size_t>(idx[row]) * C);
    BF8* dst = reinterpret_cast<BF8*>(out + static_cast<size_t>(row) * C);
    for (int i = threadIdx.x; i < nchunk; i += blockDim.x) dst[i] = src[i];
  }
}

// ------------------------------------------------------------------------------ column sum
// Two deterministic passes (no atomics, so bias gradients are reproducible bit for bit): row slab y
// writes its partial sums to part[y][C]; the second kernel adds the slabs in order and rounds.
__global__ void column_sum_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ part, int R, int C,
                                  int rows_per_block) {
  const int c2 = blockIdx.x * blockDim.x + threadIdx.x;  // pair index
  if (c2 * 2 >= C) return;
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(R, r0 + rows_per_block);
  float* acc = part + static_cast<size_t>(blockIdx.y) * C;
  float s0 = 0.f, s1 = 0.f;
  if (c2 * 2 + 1 < C && (C & 1) == 0) {
    for (int r = r0; r < r1; ++r) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + static_cast<size_t>(r) * C + c2 * 2));
      s0 += f.x;
      s1 += f.y;
    }
    acc[c2 * 2] = s0;
    acc[c2 * 2 + 1] = s1;
  } else {
    for (int r = r0; r < r1; ++r) {
      s0 += __bfloat162float(x[static_cast<size_t>(r) * C + c2 * 2]);
      if (c2 * 2 + 1 < C) s1 += __bfloat162float(x[static_cast<size_t>(r) * C + c2 * 2 + 1]);
    }
    acc[c2 * 2] = s0;
    if (c2 * 2 + 1 < C) acc[c2 * 2 + 1] = s1;
  }
}
// C % 8 == 0 and 16-byte aligned rows: 8 columns per thread, 16-byte loads, eight rows in flight
__global__ void column_sum8_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ part, int R, int C,
                                   int rows_per_block) {
  const int c8 = blockIdx.x * blockDim.x + threadIdx.x;
  if (c8 * 8 >= C) return;
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(R, r0 + rows_per_block);
  float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const __nv_bfloat16* col = x + c8 * 8;
  int r = r0;
  for (; r + 8 <= r1; r += 8) {
    BF8 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = *reinterpret_cast<const BF8*>(col + static_cast<size_t>(r + u) * C);
#pragma unroll
    for (int u = 0; u < 8; ++u) {  // rows are added in order, so the result does not depend on the unrolling
      float f[8];
      unpack8(v[u], f);
#pragma unroll
      for (int e = 0; e < 8; ++e) s[e] += f[e];
    }
  }
  for (; r < r1; ++r) {
    float f[8];
    unpack8(*reinterpret_cast<const BF8*>(col + static_cast<size_t>(r) * C), f);
#pragma unroll
    for (int e = 0; e < 8; ++e) s[e] += f[e];
  }
  float* acc = part + static_cast<size_t>(blockIdx.y) * C + c8 * 8;
  *reinterpret_cast<float4*>(acc) = make_float4(s[0], s[1], s[2], s[3]);
  *reinterpret_cast<float4*>(acc + 4) = make_float4(s[4], s[5], s[6], s[7]);
}
__global__ void column_sum_finish_kernel(const float* __restrict__ part, __nv_bfloat16* __restrict__ out, int nslab,
                                         int C) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s = 0.f;
  for (int y = 0; y < nslab; ++y) s += part[static_cast<size_t>(y) * C + c];
  out[c] = __float2bfloat16(s);
}
__global__ void f32_to_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, long n) {
  const long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __float2bfloat16(in[i]);
}

// ------------------------------------------------------------------------------ cross entropy
constexpr int CE_THREADS = 512;
__global__ void __launch_bounds__(CE_THREADS)
ce_fwd_kernel(const __nv_bfloat16* __restrict__ logits, const long* __restrict__ labels, float* __restrict__ loss,
              float* __restrict__ lse_out, long* __restrict__ pred, int R, int V, long ld) {
  __shared__ float red[32];
  __shared__ float s_max;
  __shared__ int s_arg[32];
  __shared__ float s_val[32];
  const int row = blockIdx.x;
  if (row >= R) return;
  const __nv_bfloat16* lr = logits + static_cast<size_t>(row) * ld;
  float mx = -INFINITY;
  int arg = 0;
  for (int i = threadIdx.x; i < V; i += CE_THREADS) {
    const float v = __bfloat162float(lr[i]);
    if (v > mx) {
      mx = v;
      arg = i;
    }
  }
  // argmax with lowest-index tie break
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, mx, o);
    const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
    if (ov > mx || (ov == mx && oa < arg)) {
      mx = ov;
      arg = oa;
    }
  }
  if (lane == 0) {
    s_val[warp] = mx;
    s_arg[warp] = arg;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float bm = s_val[0];
    int ba = s_arg[0];
    for (int w2 = 1; w2 < CE_THREADS / 32; ++w2)
      if (s_val[w2] > bm || (s_val[w2] == bm && s_arg[w2] < ba)) {
        bm = s_val[w2];
        ba = s_arg[w2];
      }
    s_max = bm;
    pred[row] = ba;
  }
  __syncthreads();
  const float m = s_max;
  float se = 0.f;
  for (int i = threadIdx.x; i < V; i += CE_THREADS) se += __expf(__bfloat162float(lr[i]) - m);
  se = block_sum(se, red);
  if (threadIdx.x == 0) {
    const float lse = m + logf(se);
    lse_out[row] = lse;
    const long lab = labels[row];
    (void)WX_CHK(lab == -100 || (lab >= 0 && lab < V), 4005, lab, V);  // neither a class nor the ignore index
    loss[row] = (lab >= 0 && lab < V) ? lse - __bfloat162float(lr[lab]) : 0.f;
  }
}

// in place: logits -> dlogits = (softmax - onehot) * dloss[row]; ignored rows -> 0
__global__ void __launch_bounds__(CE_THREADS)
ce_bwd_kernel(__nv_bfloat16* __restrict__ logits, const long* __restrict__ labels, const float* __restrict__ lse,
              const float* __restrict__ dloss, int R, int V, long ld) {
  const int row = blockIdx.x;
  if (row >= R) return;
  __nv_bfloat16* lr = logits + static_cast<size_t>(row) * ld;
  const long lab = labels[row];
  const bool valid = lab >= 0 && lab < V;
  const float g = valid ? dloss[row] : 0.f;
  const float l = lse[row];
  for (int i = threadIdx.x; i < V; i += CE_THREADS) {
    float p = valid ? __expf(__bfloat162float(lr[i]) - l) : 0.f;
    if (i == lab) p -= 1.f;
    lr[i] = __float2bfloat16(p * g);
  }
}

// ------------------------------------------------------------------------------ optimizer
// sum of squares of a bf16 buffer accumulated (atomically) into out[0].
constexpr int kSumsqMaxBlocks = 4096;  // scratch slots of the deterministic grid reduction
__device__ float g_sumsq_scratch[kSumsqMaxBlocks];
__device__ unsigned g_sumsq_counter = 0;

__global__ void sumsq_bf16_kernel(const __nv_bfloat16* __restrict__ g, long n, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  const long n8 = n >> 3;
  const BF8* g8 = reinterpret_cast<const BF8*>(g);
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float f[8];
    unpack8(g8[i], f);
#pragma unroll
    for (int e = 0; e < 8; ++e) s += f[e] * f[e];
  }
  for (long i = (n8 << 3) + static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const float f = __bfloat162float(g[i]);
    s += f * f;
  }
  s = block_sum(s, red);
  // Deterministic grid reduction: every block parks its sum, the block that finishes last adds them
  // in index order (no float atomics, so the gradient norm is reproducible bit for bit).
  __shared__ bool is_last;
  const unsigned nblk = gridDim.x;
  if (threadIdx.x == 0) {
    g_sumsq_scratch[blockIdx.x] = s;
    __threadfence();
    is_last = atomicInc(&g_sumsq_counter, nblk - 1) == nblk - 1;
  }
  __syncthreads();
  if (is_last) {
    __threadfence();
    float t = 0.f;
    for (unsigned i = threadIdx.x; i < nblk; i += blockDim.x) t += reinterpret_cast<volatile float*>(g_sumsq_scratch)[i];
    t = block_sum(t, red);
    if (threadIdx.x == 0) *out += t;
  }
}

// Fused: grad (bf16) * inv_accum * clip -> AdamW on fp32 master/m/v -> bf16 param.
// `hyper` (device): [0] lr, [1] beta1, [2] beta2, [3] eps, [4] weight_decay, [5] bias_corr1,
// [6] bias_corr2, [7] max_grad_norm (<=0: no clip), [8] grad_scale (1 / accumulation steps).
// `norm_sq` (device): sum of squared *unscaled* gradients over the whole model. A non-finite norm
// skips the update on every element (all ranks see the same norm, so all skip together).
__global__ void adamw_kernel(__nv_bfloat16* __restrict__ p16, float* __restrict__ p32, float* __restrict__ m,
                             float* __restrict__ v, const __nv_bfloat16* __restrict__ g, long n,
                             const float* __restrict__ hyper, const float* __restrict__ norm_sq,
                             const float* __restrict__ lr_scale_per_elem_unused) {
  const float lr = hyper[0], b1 = hyper[1], b2 = hyper[2], eps = hyper[3], wd = hyper[4], bc1 = hyper[5],
              bc2 = hyper[6], max_norm = hyper[7], gscale = hyper[8];
  const float nsq = norm_sq ? norm_sq[0] : 0.f;
  if (!(nsq == nsq) || isinf(nsq)) return;
  float scale = gscale;
  if (max_norm > 0.f && norm_sq) {
    const float gnorm = sqrtf(nsq) * gscale;
    const float coef = max_norm / (gnorm + 1e-6f);
    if (coef < 1.f) scale *= coef;
  }
  const float step_size = lr / bc1;
  const float inv_sqrt_bc2 = rsqrtf(bc2);
  const long tid0 = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long nthr = static_cast<long>(gridDim.x) * blockDim.x;
  auto update = [&](float gi, float& pi, float& mi, float& vi) {
    gi *= scale;
    pi *= (1.f - lr * wd);
    mi = b1 * mi + (1.f - b1) * gi;
    vi = b2 * vi + (1.f - b2) * gi * gi;
    pi -= step_size * mi / (sqrtf(vi) * inv_sqrt_bc2 + eps);
  };
  // four elements per thread with 16-byte accesses when every array allows it
  const bool vec = ((reinterpret_cast<uintptr_t>(p32) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v)) & 15) == 0 &&
                   ((reinterpret_cast<uintptr_t>(p16) | reinterpret_cast<uintptr_t>(g)) & 7) == 0;
  const long n4 = vec ? n >> 2 : 0;
  for (long i = tid0; i < n4; i += nthr) {
    float4 p4 = reinterpret_cast<float4*>(p32)[i], m4 = reinterpret_cast<float4*>(m)[i], v4 = reinterpret_cast<float4*>(v)[i];
    const uint2 graw = reinterpret_cast<const uint2*>(g)[i];
    const float2 g01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&graw.x));
    const float2 g23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&graw.y));
    update(g01.x, p4.x, m4.x, v4.x);
    update(g01.y, p4.y, m4.y, v4.y);
    update(g23.x, p4.z, m4.z, v4.z);
    update(g23.y, p4.w, m4.w, v4.w);
    reinterpret_cast<float4*>(m)[i] = m4;
    reinterpret_cast<float4*>(v)[i] = v4;
    reinterpret_cast<float4*>(p32)[i] = p4;
    const __nv_bfloat162 o01 = __floats2bfloat162_rn(p4.x, p4.y), o23 = __floats2bfloat162_rn(p4.z, p4.w);
    reinterpret_cast<uint2*>(p16)[i] =
        make_uint2(*reinterpret_cast<const uint32_t*>(&o01), *reinterpret_cast<const uint32_t*>(&o23));
  }
  for (long i = (n4 << 2) + tid0; i < n; i += nthr) {
    float pi = p32[i], mi = m[i], vi = v[i];
    update(__bfloat162float(g[i]), pi, mi, vi);
    m[i] = mi;
    v[i] = vi;
    p32[i] = pi;
    p16[i] = __float2bfloat16(pi);
  }
}

inline int blocks_for(long n, int threads, int cap = 0) {
  if (cap <= 0) cap = sm_count() * 16;
  long b = (n + threads - 1) / threads;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

}  // namespace

// ================================================================================ launchers
int rms_norm_fwd(const void* x, const void* w, void* y, float* rstd, const int* dest, int T, int C, float eps,
                 cudaStream_t s) {
  if (C % 8 != 0 || C > NORM_THREADS * 8 * NORM_MAX_CHUNKS) return -1;
  if (T == 0) return 0;
  if (C % 256 == 0 && C <= 2048) {  // one warp per row
    const int g = (T + 7) / 8 < sm_count() * 8 ? (T + 7) / 8 : sm_count() * 8;
    const __nv_bfloat16* xb = reinterpret_cast<const __nv_bfloat16*>(x);
    const __nv_bfloat16* wb = reinterpret_cast<const __nv_bfloat16*>(w);
    __nv_bfloat16* yb = reinterpret_cast<__nv_bfloat16*>(y);
    cudaError_t e = cudaSuccess;
    switch (C / 256) {
#define WX_CASE(n)                                                                                                        \
  case n:                                                                                                                 \
    e = (T <= 1024) ? launch_kernel(rms_norm_fwd_warp_kernel<n, true>, dim3(g), dim3(256), 0, s, xb, wb, yb, rstd, dest, T, eps) \
                    : launch_kernel(rms_norm_fwd_warp_kernel<n, false>, dim3(g), dim3(256), 0, s, xb, wb, yb, rstd, dest, T, eps); \
    break;
      WX_CASE(1) WX_CASE(2) WX_CASE(3) WX_CASE(4) WX_CASE(5) WX_CASE(6) WX_CASE(7) WX_CASE(8)
#undef WX_CASE
    }
    return static_cast<int>(e);
  }
  const int grid = T < sm_count() * 8 ? T : sm_count() * 8;
  rms_norm_fwd_kernel<<<grid, NORM_THREADS, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x),
                                                     reinterpret_cast<const __nv_bfloat16*>(w),
                                                     reinterpret_cast<__nv_bfloat16*>(y), rstd, dest, T, C, eps);
  return static_cast<int>(cudaGetLastError());
}

int rms_norm_bwd_blocks(int T) { return T < sm_count() * 2 ? (T > 0 ? T : 1) : sm_count() * 2; }

int rms_norm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const int* dest, void* dx,
                 float* dw_partial, void* dw, int T, int C, cudaStream_t s, const void* add) {
  const __nv_bfloat16* addb = reinterpret_cast<const __nv_bfloat16*>(add);
  if (C % 8 != 0 || C > NORM_THREADS * 8 * NORM_MAX_CHUNKS) return -1;
  const int grid = rms_norm_bwd_blocks(T);
  if (C % 256 == 0 && C <= 2048) {  // one warp per row; the number of partial rows is the same
    const __nv_bfloat16* dyb = reinterpret_cast<const __nv_bfloat16*>(dy);
    const __nv_bfloat16* xb = reinterpret_cast<const __nv_bfloat16*>(x);
    const __nv_bfloat16* wb = reinterpret_cast<const __nv_bfloat16*>(w);
    __nv_bfloat16* dxb = reinterpret_cast<__nv_bfloat16*>(dx);
    switch (C / 256) {
#define WX_CASE(n) case n: rms_norm_bwd_warp_kernel<n><<<grid, 256, 0, s>>>(dyb, xb, wb, rstd, dest, dxb, dw_partial, T, addb); break;
      WX_CASE(1) WX_CASE(2) WX_CASE(3) WX_CASE(4) WX_CASE(5) WX_CASE(6) WX_CASE(7) WX_CASE(8)
#undef WX_CASE
    }
    reduce_partials_kernel<<<(C + 255) / 256, 256, 0, s>>>(dw_partial, reinterpret_cast<__nv_bfloat16*>(dw), grid, C);
    return static_cast<int>(cudaGetLastError());
  }
  rms_norm_bwd_kernel<<<grid, NORM_THREADS, 0, s>>>(
      reinterpret_cast<const __nv_bfloat16*>(dy), reinterpret_cast<const __nv_bfloat16*>(x),
      reinterpret_cast<const __nv_bfloat16*>(w), rstd, dest, reinterpret_cast<__nv_bfloat16*>(dx), dw_partial, T, C, addb);
  reduce_partials_kernel<<<(C + 255) / 256, 256, 0, s>>>(dw_partial, reinterpret_cast<__nv_bfloat16*>(dw), grid, C);
  return static_cast<int>(cudaGetLastError());
}

int swiglu_bwd(const void* dh, const void* gu, void* dgu, int R, int width_gu, long ld_dh, long ld_gu,
               cudaStream_t s) {
  if (width_gu % 32 != 0 || ld_dh % 8 != 0 || ld_gu % 8 != 0) return -1;
  const int nblk = width_gu / 32;
  const long total = static_cast<long>(R) * nblk * 2;
  if (total == 0) return 0;
  swiglu_bwd_kernel<<<blocks_for(total, 256, sm_count() * 32), 256, 0, s>>>(
      reinterpret_cast<const __nv_bfloat16*>(dh), reinterpret_cast<const __nv_bfloat16*>(gu),
      reinterpret_cast<__nv_bfloat16*>(dgu), R, nblk, ld_dh, ld_gu);
  return static_cast<int>(cudaGetLastError());
}

int rope_qk(const void* in, void* out, const float* cos_t, const float* sin_t, int T, int W, int n_rot, int D,
            int inverse, cudaStream_t s) {
  if (D % 16 != 0 || W % 8 != 0 || n_rot * D > W) return -1;
  const long total = static_cast<long>(D / 16) * T;  // D/16 threads per token
  if (total == 0) return 0;
  // few tokens: too little parallelism with one thread per 8-channel column; head dims that are not a
  // multiple of 128 (ViT: 80): a token's threads would read 80-byte pieces
  // in place (in == out): every thread reads its rotation pairs before it writes them, and the columns that are not
  // rotated (v) need no copy, which saves a third of the traffic of a q|k|v buffer with as many v as q heads
  const int copy_rest = (in != out) ? 1 : 0;
  if (total < static_cast<long>(sm_count()) * 256 || D % 128 != 0) {
    const long per_row = static_cast<long>(n_rot) * (D / 16) + (copy_rest ? (W - n_rot * D) / 8 : 0);
    rope_qk_chunk_kernel<<<static_cast<unsigned>((per_row * T + 255) / 256), 256, 0, s>>>(
        reinterpret_cast<const __nv_bfloat16*>(in), reinterpret_cast<__nv_bfloat16*>(out), cos_t, sin_t, T, W, n_rot, D,
        inverse, copy_rest);
    return static_cast<int>(cudaGetLastError());
  }
  rope_qk_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, s>>>(
      reinterpret_cast<const __nv_bfloat16*>(in), reinterpret_cast<__nv_bfloat16*>(out), cos_t, sin_t, T, W, n_rot, D,
      inverse, copy_rest);
  return static_cast<int>(cudaGetLastError());
}

int route_plan(const int* types, int T, int E, int rows, int* dest, int* seg, int* segk, int* inv, cudaStream_t s) {
  if (E < 1 || E > ROUTE_MAX_E) return -1;
  route_plan_kernel<<<1, ROUTE_THREADS, 0, s>>>(types, T, E, rows, dest, seg, segk, inv);
  return static_cast<int>(cudaGetLastError());
}

int permute_rows(const void* x, const int* dest, void* out, int T, int C, cudaStream_t s, int out_rows) {
  if (C % 8 != 0) return -1;
  if (T == 0) return 0;
  permute_rows_kernel<<<T < sm_count() * 16 ? T : sm_count() * 16, 128, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x), dest,
                                                                  reinterpret_cast<__nv_bfloat16*>(out), T, C, out_rows);
  return static_cast<int>(cudaGetLastError());
}

int gather_rows(const void* x, const int* idx, void* out, int T, int C, cudaStream_t s, int src_rows) {
  if (C % 8 != 0) return -1;
  if (T == 0) return 0;
  gather_rows_kernel<<<T < sm_count() * 16 ? T : sm_count() * 16, 128, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x), idx,
                                                                 reinterpret_cast<__nv_bfloat16*>(out), T, C, src_rows);
  return static_cast<int>(cudaGetLastError());
}

int column_sum_slabs(int R) {
  int ysplit = (R + 63) / 64;  // 64-row slabs: enough blocks to keep every SM's memory pipe full
  if (ysplit > 512) ysplit = 512;
  return ysplit < 1 ? 1 : ysplit;
}

int column_sum(const void* x, float* partials, void* out_bf16, int R, int C, cudaStream_t s) {
  if (C == 0) return 0;
  if (R == 0) return static_cast<int>(cudaMemsetAsync(out_bf16, 0, static_cast<size_t>(C) * 2, s));
  const int pairs = (C + 1) / 2;
  const int ysplit = column_sum_slabs(R);
  const int rpb = (R + ysplit - 1) / ysplit;
  if (C % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    dim3 grid8((C / 8 + 63) / 64, ysplit);
    column_sum8_kernel<<<grid8, 64, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x), partials, R, C, rpb);
  } else {
    dim3 grid((pairs + 127) / 128, ysplit);
    column_sum_kernel<<<grid, 128, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x), partials, R, C, rpb);
  }
  column_sum_finish_kernel<<<(C + 255) / 256, 256, 0, s>>>(partials, reinterpret_cast<__nv_bfloat16*>(out_bf16), ysplit, C);
  return static_cast<int>(cudaGetLastError());
}

int ce_fwd(const void* logits, const long* labels, float* loss, float* lse, long* pred, int R, int V, long ld,
           cudaStream_t s) {
  if (R == 0) return 0;
  ce_fwd_kernel<<<R, CE_THREADS, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(logits), labels, loss, lse, pred, R, V,
                                         ld);
  return static_cast<int>(cudaGetLastError());
}

int ce_bwd(void* logits, const long* labels, const float* lse, const float* dloss, int R, int V, long ld,
           cudaStream_t s) {
  if (R == 0) return 0;
  ce_bwd_kernel<<<R, CE_THREADS, 0, s>>>(reinterpret_cast<__nv_bfloat16*>(logits), labels, lse, dloss, R, V, ld);
  return static_cast<int>(cudaGetLastError());
}

int sumsq_bf16(const void* g, long n, float* out, cudaStream_t s) {
  if (n == 0) return 0;
  sumsq_bf16_kernel<<<blocks_for(n / 8 + 1, 256, sm_count() * 8 < kSumsqMaxBlocks ? sm_count() * 8 : kSumsqMaxBlocks), 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(g), n,
                                                                        out);
  return static_cast<int>(cudaGetLastError());
}

int adamw_step(void* p16, float* p32, float* m, float* v, const void* g, long n, const float* hyper,
               const float* norm_sq, cudaStream_t s) {
  if (n == 0) return 0;
  adamw_kernel<<<blocks_for(n, 256, sm_count() * 16), 256, 0, s>>>(reinterpret_cast<__nv_bfloat16*>(p16), p32, m, v,
                                                            reinterpret_cast<const __nv_bfloat16*>(g), n, hyper,
                                                            norm_sq, nullptr);
  return static_cast<int>(cudaGetLastError());
}

WX_CHK_DEFINE_READER(kernels_check_read)

}  // namespace wx
