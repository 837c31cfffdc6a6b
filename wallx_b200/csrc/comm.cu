// NVLink / NVSwitch data plane of the sharded optimizer: flag barrier, gradient reduce-scatter
// (peer loads, fp32 sum), parameter all-gather (peer stores), small-vector all-reduce, AdamW on
// fp32 shards. The reference delegates all of this to NCCL through accelerate/FSDP2
// (train_qact.py:42-49, qwen_vl_act_trainer.py:335-337, 609-611).
//
// NVSwitch gives every peer full bandwidth, so each rank pulls its shard from all peers at once
// (one-shot reduce-scatter) and pushes its updated shard to all peers at once (one-shot
// all-gather); there is no ring. Waits on peer flags are bounded: after the caller's limit (2 s by
// default, ten minutes at most) the kernel records an error status and returns.
#include "comm.h"
#include "check.cuh"
#include "devinfo.h"

#include <cuda_bf16.h>

namespace wx {

namespace {

__device__ __forceinline__ uint64_t gtimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void symm_barrier_kernel(PeerPtrs flags, int rank, int world, int epoch, int* status, uint64_t limit_ns) {
  const int p = threadIdx.x;
  if (p >= world) return;
  if (!WX_CHK(rank >= 0 && rank < world && world <= kMaxPeers && epoch > 0 && flags.p[p] != nullptr, 6003, rank, epoch)) {
    atomicExch(status, 15);
    return;
  }
  __threadfence_system();
  st_release_sys(reinterpret_cast<int*>(flags.p[p]) + rank, epoch);
  const int* mine = reinterpret_cast<const int*>(flags.p[rank]) + p;
  const uint64_t t0 = gtimer_ns();
  unsigned it = 0;
  while (ld_acquire_sys(mine) < epoch) {
    if (((++it) & 1023u) == 0u && gtimer_ns() - t0 > limit_ns) {
      atomicExch(status, 16 + p);  // peer p never arrived
      return;
    }
  }
}

struct alignas(16) BF8 {
  __nv_bfloat162 v[4];
};

constexpr int kRsMaxBlocks = 8192;
__device__ float g_rs_scratch[kRsMaxBlocks];
__device__ unsigned g_rs_counter = 0;

__global__ void __launch_bounds__(256)
rs_reduce_kernel(PeerPtrs grads, const ShardDesc* __restrict__ table, int world, float* __restrict__ out,
                 float* __restrict__ sumsq) {
  __shared__ float red[8];
  const ShardDesc d = table[blockIdx.y];
  // 16-byte vector loads and stores: offsets and lengths in whole groups of eight bf16 / four fp32
  const long n8 = WX_CHK(d.n >= 0 && ((d.n | d.arena_off) & 7) == 0 && (d.out_off & 3) == 0 && world >= 1 && world <= kMaxPeers,
                         6001, d.arena_off, d.n) ? d.n >> 3 : 0;
  float ss = 0.f;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    // all ranks' loads are issued before the first add (peer loads have microseconds of latency)
    BF8 x[kMaxPeers];
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)
      if (r < world)
        x[r] = reinterpret_cast<const BF8*>(reinterpret_cast<const __nv_bfloat16*>(grads.p[r]) + d.arena_off)[i];
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r) {
      if (r < world) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(x[r].v[e]);
          acc[2 * e] += f.x;
          acc[2 * e + 1] += f.y;
        }
      }
    }
    float4* o = reinterpret_cast<float4*>(out + d.out_off + i * 8);
    o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += acc[e] * acc[e];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  // Deterministic grid reduction (see sumsq_bf16_kernel): the last block adds the parked sums in order.
  __shared__ bool is_last;
  const unsigned nblk = gridDim.x * gridDim.y;
  const unsigned bid = blockIdx.y * gridDim.x + blockIdx.x;
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += red[w];
    g_rs_scratch[bid] = t;
    __threadfence();
    is_last = atomicInc(&g_rs_counter, nblk - 1) == nblk - 1;
  }
  __syncthreads();
  if (is_last) {
    __threadfence();
    float t = 0.f;
    for (unsigned i = threadIdx.x; i < nblk; i += blockDim.x) t += reinterpret_cast<volatile float*>(g_rs_scratch)[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = t;
    __syncthreads();
    if (threadIdx.x == 0) {
      float u = 0.f;
      for (int w = 0; w < 8; ++w) u += red[w];
      *sumsq += u;  // launches that share `sumsq` must be ordered by their streams
    }
  }
}

__global__ void __launch_bounds__(256)
ag_push_kernel(PeerPtrs params, const ShardDesc* __restrict__ table, int rank, int world) {
  const ShardDesc d = table[blockIdx.y];
  const long n8 = WX_CHK(d.n >= 0 && ((d.n | d.arena_off) & 7) == 0 && rank >= 0 && rank < world && world <= kMaxPeers, 6002,
                         d.arena_off, d.n) ? d.n >> 3 : 0;
  const BF8* src = reinterpret_cast<const BF8*>(reinterpret_cast<const __nv_bfloat16*>(params.p[rank]) + d.arena_off);
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const BF8 x = src[i];
#pragma unroll 1
    for (int r = 0; r < world; ++r) {
      if (r == rank) continue;
      reinterpret_cast<BF8*>(reinterpret_cast<__nv_bfloat16*>(params.p[r]) + d.arena_off)[i] = x;
    }
  }
}

// Same result through the NVSwitch multicast mapping of the parameter arena: one multimem.st per 16 bytes is
// replicated by the switch into every GPU's copy (this rank's included), so each byte leaves this GPU once instead
// of once per peer. `mc_base` is the multicast address of the arena, `local` this rank's own mapping (the source).
__global__ void __launch_bounds__(256)
ag_push_mc_kernel(void* mc_base, const void* local, const ShardDesc* __restrict__ table) {
  const ShardDesc d = table[blockIdx.y];
  const long n8 = WX_CHK(d.n >= 0 && ((d.n | d.arena_off) & 7) == 0 && mc_base != nullptr, 6004, d.arena_off, d.n) ? d.n >> 3 : 0;
  const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const __nv_bfloat16*>(local) + d.arena_off);
  float4* dst = reinterpret_cast<float4*>(reinterpret_cast<__nv_bfloat16*>(mc_base) + d.arena_off);
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const float4 x = src[i];
    asm volatile("multimem.st.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + i), "f"(x.x), "f"(x.y), "f"(x.z), "f"(x.w)
                 : "memory");
  }
}

__global__ void small_allreduce_write_kernel(PeerPtrs scratch, const float* __restrict__ vals, int n, int rank,
                                             int world) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = vals[i];
  for (int r = 0; r < world; ++r) reinterpret_cast<float*>(scratch.p[r])[static_cast<long>(rank) * n + i] = v;
}
__global__ void small_allreduce_sum_kernel(const float* __restrict__ mine, float* __restrict__ out, int n, int world) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s = 0.f;
  for (int r = 0; r < world; ++r) s += mine[static_cast<long>(r) * n + i];
  out[i] = s;
}

__global__ void adamw_f32g_kernel(__nv_bfloat16* __restrict__ p16, float* __restrict__ p32, float* __restrict__ m,
                                  float* __restrict__ v, const float* __restrict__ g, long n,
                                  const float* __restrict__ hyper, const float* __restrict__ norm_sq) {
  const float lr = hyper[0], b1 = hyper[1], b2 = hyper[2], eps = hyper[3], wd = hyper[4], bc1 = hyper[5],
              bc2 = hyper[6], max_norm = hyper[7], gscale = hyper[8];
  const float nsq = norm_sq ? norm_sq[0] : 0.f;
  if (!(nsq == nsq) || isinf(nsq)) return;
  float scale = gscale;
  if (max_norm > 0.f && norm_sq) {
    const float coef = max_norm / (sqrtf(nsq) * gscale + 1e-6f);
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
  const bool vec = ((reinterpret_cast<uintptr_t>(p32) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v) |
                     reinterpret_cast<uintptr_t>(g)) & 15) == 0 && (reinterpret_cast<uintptr_t>(p16) & 7) == 0;
  const long n4 = vec ? n >> 2 : 0;
  for (long i = tid0; i < n4; i += nthr) {
    float4 p4 = reinterpret_cast<float4*>(p32)[i], m4 = reinterpret_cast<float4*>(m)[i], v4 = reinterpret_cast<float4*>(v)[i];
    const float4 g4 = reinterpret_cast<const float4*>(g)[i];
    update(g4.x, p4.x, m4.x, v4.x);
    update(g4.y, p4.y, m4.y, v4.y);
    update(g4.z, p4.z, m4.z, v4.z);
    update(g4.w, p4.w, m4.w, v4.w);
    reinterpret_cast<float4*>(m)[i] = m4;
    reinterpret_cast<float4*>(v)[i] = v4;
    reinterpret_cast<float4*>(p32)[i] = p4;
    const __nv_bfloat162 o01 = __floats2bfloat162_rn(p4.x, p4.y), o23 = __floats2bfloat162_rn(p4.z, p4.w);
    reinterpret_cast<uint2*>(p16)[i] =
        make_uint2(*reinterpret_cast<const uint32_t*>(&o01), *reinterpret_cast<const uint32_t*>(&o23));
  }
  for (long i = (n4 << 2) + tid0; i < n; i += nthr) {
    float pi = p32[i], mi = m[i], vi = v[i];
    update(g[i], pi, mi, vi);
    m[i] = mi;
    v[i] = vi;
    p32[i] = pi;
    p16[i] = __float2bfloat16(pi);
  }
}

}  // namespace

WX_CHK_DEFINE_READER(comm_check_read)

int symm_barrier(const PeerPtrs& flags, int rank, int world, int epoch, int* status, cudaStream_t s, long timeout_ms) {
  if (world < 1 || world > kMaxPeers) return -1;
  if (timeout_ms < 1) timeout_ms = 1;
  if (timeout_ms > 600000) timeout_ms = 600000;  // always bounded: ten minutes at most
  symm_barrier_kernel<<<1, 32, 0, s>>>(flags, rank, world, epoch, status, static_cast<uint64_t>(timeout_ms) * 1000000ull);
  return static_cast<int>(cudaGetLastError());
}

int rs_reduce(const PeerPtrs& grads, const ShardDesc* table_dev, int nbuf, int world, float* out, float* sumsq,
              cudaStream_t s) {
  if (nbuf == 0) return 0;
  // about 16 resident blocks per SM in total, whatever the number of buffers
  int gx = (sm_count() * 16 + nbuf - 1) / nbuf;
  gx = gx < 8 ? 8 : gx;
  if (static_cast<long>(gx) * nbuf > kRsMaxBlocks) gx = kRsMaxBlocks / nbuf;
  if (gx < 1) return -1;
  rs_reduce_kernel<<<dim3(gx, nbuf), 256, 0, s>>>(grads, table_dev, world, out, sumsq);
  return static_cast<int>(cudaGetLastError());
}

int ag_push(const PeerPtrs& params, const ShardDesc* table_dev, int nbuf, int rank, int world, cudaStream_t s) {
  if (nbuf == 0 || world == 1) return 0;
  int gx = (sm_count() * 16 + nbuf - 1) / nbuf;
  gx = gx < 8 ? 8 : gx;
  ag_push_kernel<<<dim3(gx, nbuf), 256, 0, s>>>(params, table_dev, rank, world);
  return static_cast<int>(cudaGetLastError());
}

int ag_push_multicast(void* mc_base, const void* local_base, const ShardDesc* table_dev, int nbuf, cudaStream_t s) {
  if (nbuf == 0) return 0;
  if (mc_base == nullptr || local_base == nullptr) return -1;
  int gx = (sm_count() * 16 + nbuf - 1) / nbuf;
  gx = gx < 8 ? 8 : gx;
  ag_push_mc_kernel<<<dim3(gx, nbuf), 256, 0, s>>>(mc_base, local_base, table_dev);
  return static_cast<int>(cudaGetLastError());
}

int small_allreduce_write(const PeerPtrs& scratch, const float* vals, int n, int rank, int world, cudaStream_t s) {
  small_allreduce_write_kernel<<<(n + 127) / 128, 128, 0, s>>>(scratch, vals, n, rank, world);
  return static_cast<int>(cudaGetLastError());
}
int small_allreduce_sum(const float* my_scratch, float* out, int n, int world, cudaStream_t s) {
  small_allreduce_sum_kernel<<<(n + 127) / 128, 128, 0, s>>>(my_scratch, out, n, world);
  return static_cast<int>(cudaGetLastError());
}

int adamw_step_f32g(void* p16, float* p32, float* m, float* v, const float* g, long n, const float* hyper,
                    const float* norm_sq, cudaStream_t s) {
  if (n == 0) return 0;
  long b = (n + 255) / 256;
  if (b > static_cast<long>(sm_count()) * 16) b = static_cast<long>(sm_count()) * 16;
  adamw_f32g_kernel<<<static_cast<unsigned>(b), 256, 0, s>>>(reinterpret_cast<__nv_bfloat16*>(p16), p32, m, v, g, n,
                                                             hyper, norm_sq);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace wx
