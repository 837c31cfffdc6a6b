// Kernels of the cached decode / denoise step (a few new rows per sequence against a key-value cache), sm_100a.
//
//   rope_cache_kernel   rotary on the q and k heads of a packed q|k|v buffer; q is rotated in place, the rotated k
//                       and the v columns go straight to the rows' cache slots (one launch instead of a rotary
//                       kernel plus an index copy).
//   attn_decode_kernel  attention of few query rows over the cache. With 32 query rows the tensor-core kernel of
//                       attention.cu has 16 CTAs that each walk the keys tile by tile, latency after latency (15 us
//                       measured); here one CTA serves one query row and one key-value head, stages a block of 128
//                       keys and values in shared memory once for the query heads that share them, and a warp per
//                       query head does the scores (one key per lane), an online softmax and the weighted sum of
//                       values (four channels per lane) in fp32.
//
// Reference parity: the reference re-runs the whole sequence through flash-attn at every denoise step
// (wall_x/model/qwen2_5_based/modeling_qwen2_5_vl_act.py:1906-1952); the masking rule is that of attention.cu
// (bottom-right aligned causal limit per query row, plus flagged queries seeing flagged keys).
#include "decode.h"
#include "check.cuh"
#include "devinfo.h"
#include "launch.h"
#include "ptx.cuh"

#include <atomic>

#include <cuda_bf16.h>

namespace wx {

namespace {
std::atomic<bool> g_pdl{false};
}  // namespace
bool pdl_enabled() { return g_pdl.load(std::memory_order_relaxed); }
void pdl_set(bool on) { g_pdl.store(on, std::memory_order_relaxed); }

namespace {

struct alignas(16) Pack8 {
  __nv_bfloat162 v[4];
};

// ------------------------------------------------------------------------------------------------ rotary + cache
__global__ void __launch_bounds__(256)
rope_cache_kernel(__nv_bfloat16* qkv, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                  const long* __restrict__ cache_rows, __nv_bfloat16* cache, int T, int W, int hq, int hkv, int D,
                  long ld_cache, long cache_nrows) {
  const int half = D >> 1;
  const int cph = half >> 3;                 // 8-channel chunks per rotated head (each covers both halves)
  const int rot_chunks = (hq + hkv) * cph;
  const int v_chunks = (hkv * D) >> 3;
  const int per_row = rot_chunks + v_chunks;
  const long idx = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
  pdl_wait();
  pdl_launch_dependents();
  if (idx >= static_cast<long>(T) * per_row) return;
  const int t = static_cast<int>(idx / per_row);
  const int c = static_cast<int>(idx - static_cast<long>(t) * per_row);
  __nv_bfloat16* row = qkv + static_cast<size_t>(t) * W;
  const long crow = cache_rows[t];
  if (!WX_CHK(crow >= 0 && crow < cache_nrows, 7001, crow, cache_nrows)) return;
  __nv_bfloat16* dst_row = cache + crow * ld_cache;
  if (c >= rot_chunks) {  // v: copy to the cache
    const int off = (c - rot_chunks) * 8;
    *reinterpret_cast<Pack8*>(dst_row + hkv * D + off) = *reinterpret_cast<const Pack8*>(row + (hq + hkv) * D + off);
    return;
  }
  const int h = c / cph;
  const int d0 = (c - h * cph) * 8;
  const Pack8 pa = *reinterpret_cast<const Pack8*>(row + h * D + d0);
  const Pack8 pb = *reinterpret_cast<const Pack8*>(row + h * D + half + d0);
  const float* cs = cos_t + static_cast<size_t>(t) * D;
  const float* sn = sin_t + static_cast<size_t>(t) * D;
  float c1[8], s1[8], c2[8], s2[8];
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    *reinterpret_cast<float4*>(c1 + 4 * q) = *reinterpret_cast<const float4*>(cs + d0 + 4 * q);
    *reinterpret_cast<float4*>(s1 + 4 * q) = *reinterpret_cast<const float4*>(sn + d0 + 4 * q);
    *reinterpret_cast<float4*>(c2 + 4 * q) = *reinterpret_cast<const float4*>(cs + half + d0 + 4 * q);
    *reinterpret_cast<float4*>(s2 + 4 * q) = *reinterpret_cast<const float4*>(sn + half + d0 + 4 * q);
  }
  Pack8 oa, ob;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 a = __bfloat1622float2(pa.v[e]);
    const float2 b = __bfloat1622float2(pb.v[e]);
    oa.v[e] = __floats2bfloat162_rn(a.x * c1[2 * e] - b.x * s1[2 * e], a.y * c1[2 * e + 1] - b.y * s1[2 * e + 1]);
    ob.v[e] = __floats2bfloat162_rn(b.x * c2[2 * e] + a.x * s2[2 * e], b.y * c2[2 * e + 1] + a.y * s2[2 * e + 1]);
  }
  __nv_bfloat16* dst = (h < hq) ? row + h * D : dst_row + (h - hq) * D;  // q in place, k to its cache slot
  *reinterpret_cast<Pack8*>(dst + d0) = oa;
  *reinterpret_cast<Pack8*>(dst + half + d0) = ob;
}

// ------------------------------------------------------------------------------------------------ attention
constexpr int kDecD = 128;           // head dimension served
constexpr int kDecBlock = 128;       // keys per shared-memory block
constexpr int kDecKPitch = 272;      // bytes per staged key row: 256 + 16, so that lanes reading different rows 16
                                     // bytes at a time fall into different banks
constexpr int kDecVPitch = 256;
constexpr int kDecMaxWarps = 4;
constexpr int kDecMaxSplits = 8;     // CTAs of a cluster that share the key blocks of one query row
constexpr int kDecComb = kDecD + 4;  // floats a warp hands to the combine step: its 128 channels, then m and l

// About 70 KB, so that three CTAs fit on an SM: a CTA loads a block and then works on it, and the other CTAs of the
// SM fill the time of its loads.
struct DecSmem {
  uint8_t k[kDecBlock * kDecKPitch];
  uint8_t v[kDecBlock * kDecVPitch];
  float p[kDecMaxWarps][kDecBlock];
  float comb[kDecMaxWarps][kDecComb];
  int vis[kDecBlock];
};

// 16-byte asynchronous copy global -> shared; `bytes` = 0 writes zeros (rows past the key range)
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, int bytes) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// Grid: x = query row * splits + split (a cluster of `splits` CTAs per row), y = key-value head, z = group of `warps`
// query heads. CTA `split` of a cluster takes the key blocks split, split + splits, ... of the row's key range; its
// warps (one query head each) keep a running maximum, sum and weighted value sum, and leave them in shared memory.
// After a cluster barrier the first CTA of the cluster merges the partial results in split order through distributed
// shared memory and stores the row.
__global__ void __launch_bounds__(kDecMaxWarps * 32)
attn_decode_kernel(const __nv_bfloat16* __restrict__ q, long ldq, const __nv_bfloat16* __restrict__ k, long ldk,
                   const __nv_bfloat16* __restrict__ v, long ldv, const int4* __restrict__ qtab,
                   const int4* __restrict__ ktab, __nv_bfloat16* __restrict__ out, long ldo, int Tq, int Tk, int hq,
                   int hkv, float scale_log2e, int warps, int splits) {
  extern __shared__ uint8_t dec_smem_raw[];
  DecSmem& sm = *reinterpret_cast<DecSmem*>((reinterpret_cast<uintptr_t>(dec_smem_raw) + 15) & ~uintptr_t(15));
  const int row = static_cast<int>(blockIdx.x) / splits;
  const int split = static_cast<int>(blockIdx.x) - row * splits;  // = %cluster_ctarank
  const int kvh = static_cast<int>(blockIdx.y);
  const int rep = hq / hkv;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int head_in_group = static_cast<int>(blockIdx.z) * warps + warp;
  const bool active = head_in_group < rep && warp < warps;  // other warps only help with the staging
  const int head = kvh * rep + head_in_group;
  pdl_wait();
  pdl_launch_dependents();
  const int4 qt = qtab[row];
  const int k_lo = max(qt.x, 0), k_hi = min(qt.y, Tk), k_lim = qt.z, qflag = qt.w;

  // this head's query vector, all of it in every lane (lanes own keys in the score pass)
  __nv_bfloat162 qv[kDecD / 2];
  if (active) {
    const Pack8* qp = reinterpret_cast<const Pack8*>(q + static_cast<size_t>(row) * ldq + head * kDecD);
#pragma unroll
    for (int i = 0; i < kDecD / 8; ++i) {
      const Pack8 x = qp[i];
#pragma unroll
      for (int e = 0; e < 4; ++e) qv[4 * i + e] = x.v[e];
    }
  }
  float m = -INFINITY, l = 0.f;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const int nthreads = static_cast<int>(blockDim.x);

  for (int base = k_lo + split * kDecBlock; base < k_hi; base += splits * kDecBlock) {
    __syncthreads();  // everybody is done with the block before this one
    for (int i = threadIdx.x; i < kDecBlock * 16; i += nthreads) {
      const int r = i >> 4, piece = i & 15;
      const int j = base + r;
      const bool in = j < k_hi;
      const size_t jj = in ? static_cast<size_t>(j) : 0;  // a valid address even when nothing is read from it
      cp_async16(sm.k + r * kDecKPitch + piece * 16, k + jj * ldk + kvh * kDecD + piece * 8, in ? 16 : 0);
      cp_async16(sm.v + r * kDecVPitch + piece * 16, v + jj * ldv + kvh * kDecD + piece * 8, in ? 16 : 0);
    }
    for (int r = threadIdx.x; r < kDecBlock; r += nthreads) {
      const int j = base + r;
      int vis = 0;
      if (j < k_hi) vis = (j <= k_lim) || (qflag != 0 && (ktab[j].w & 1) != 0);
      sm.vis[r] = vis;
    }
    cp_async_wait_all();
    __syncthreads();  // the block (every thread's copies) has landed
    if (!active) continue;
    // ---- scores: lane owns keys lane, lane + 32, lane + 64, lane + 96 of the block (four independent sums)
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    const uint8_t* kr = sm.k + lane * kDecKPitch;
#pragma unroll
    for (int cidx = 0; cidx < 16; ++cidx) {
      float qf[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(qv[4 * cidx + e]);
        qf[2 * e] = f.x;
        qf[2 * e + 1] = f.y;
      }
#pragma unroll
      for (int r4 = 0; r4 < 4; ++r4) {
        const uint4 x = *reinterpret_cast<const uint4*>(kr + r4 * 32 * kDecKPitch + cidx * 16);
        const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 kf = __bfloat1622float2(xb[e]);
          s[r4] = fmaf(kf.x, qf[2 * e], s[r4]);
          s[r4] = fmaf(kf.y, qf[2 * e + 1], s[r4]);
        }
      }
    }
#pragma unroll
    for (int r4 = 0; r4 < 4; ++r4) s[r4] = sm.vis[lane + 32 * r4] ? s[r4] * scale_log2e : -INFINITY;
    float bm = fmaxf(fmaxf(s[0], s[1]), fmaxf(s[2], s[3]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, o));
    if (bm == -INFINITY) continue;  // nothing of this block is visible (uniform over the warp)
    const float m_new = fmaxf(m, bm);
    const float corr = (m == -INFINITY) ? 0.f : exp2f(m - m_new);
    float ps = 0.f;
#pragma unroll
    for (int r4 = 0; r4 < 4; ++r4) {
      const float pj = (s[r4] == -INFINITY) ? 0.f : exp2f(s[r4] - m_new);
      sm.p[warp][lane + 32 * r4] = pj;
      ps += pj;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
    l = l * corr + ps;
    m = m_new;
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[e] *= corr;
    __syncwarp();
    // ---- weighted values: lane owns channels 4 * lane .. 4 * lane + 3
    const int nvalid = min(kDecBlock, k_hi - base);
    const uint8_t* vr = sm.v + lane * 8;
#pragma unroll 4
    for (int j = 0; j < nvalid; ++j) {
      const float pj = sm.p[warp][j];
      const uint2 x = *reinterpret_cast<const uint2*>(vr + j * kDecVPitch);
      const float2 v01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x.x));
      const float2 v23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x.y));
      acc[0] = fmaf(pj, v01.x, acc[0]);
      acc[1] = fmaf(pj, v01.y, acc[1]);
      acc[2] = fmaf(pj, v23.x, acc[2]);
      acc[3] = fmaf(pj, v23.y, acc[3]);
    }
    __syncwarp();
  }

  // ---- hand the partial result to the cluster's first CTA and merge there, in split order
  if (active) {
    *reinterpret_cast<float4*>(&sm.comb[warp][lane * 4]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    if (lane == 0) {
      sm.comb[warp][kDecD] = m;
      sm.comb[warp][kDecD + 1] = l;
    }
  }
  __syncthreads();
  if (splits > 1) {
    cluster_arrive();
    cluster_wait();
  }
  if (active && split == 0) {
    const uint32_t mine = smem_u32(&sm.comb[warp][0]);
    float ms[kDecMaxSplits];
    float m_all = -INFINITY;
#pragma unroll
    for (int sp = 0; sp < kDecMaxSplits; ++sp) {
      ms[sp] = -INFINITY;
      if (sp < splits) {
        const float4 ml = ld_cluster_f32x4(mapa_u32(mine + kDecD * 4, static_cast<uint32_t>(sp)));
        ms[sp] = ml.x;
        m_all = fmaxf(m_all, ml.x);
      }
    }
    float o4[4] = {0.f, 0.f, 0.f, 0.f};
    float l_all = 0.f;
#pragma unroll
    for (int sp = 0; sp < kDecMaxSplits; ++sp) {
      if (sp < splits && ms[sp] != -INFINITY) {
        const uint32_t peer = mapa_u32(mine, static_cast<uint32_t>(sp));
        const float w = exp2f(ms[sp] - m_all);
        const float4 a = ld_cluster_f32x4(peer + lane * 16);
        const float4 ml = ld_cluster_f32x4(peer + kDecD * 4);
        o4[0] = fmaf(w, a.x, o4[0]);
        o4[1] = fmaf(w, a.y, o4[1]);
        o4[2] = fmaf(w, a.z, o4[2]);
        o4[3] = fmaf(w, a.w, o4[3]);
        l_all = fmaf(w, ml.y, l_all);
      }
    }
    const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
    uint2 o;
    *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(o4[0] * inv, o4[1] * inv);
    *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(o4[2] * inv, o4[3] * inv);
    *reinterpret_cast<uint2*>(out + static_cast<size_t>(row) * ldo + head * kDecD + lane * 4) = o;
  }
  if (splits > 1) {  // nobody leaves while the first CTA may still read its partial result
    __syncthreads();
    cluster_arrive();
    cluster_wait();
  }
}

}  // namespace

int rope_cache(void* qkv, const float* cos_t, const float* sin_t, const long* cache_rows, void* cache, int T, int W,
               int hq, int hkv, int D, long ld_cache, long cache_nrows, cudaStream_t s) {
  if (D % 16 != 0 || W % 8 != 0 || (hq + 2 * hkv) * D != W || ld_cache % 8 != 0 || ld_cache < 2L * hkv * D) return -1;
  if (T == 0) return 0;
  const long per_row = static_cast<long>(hq + hkv) * (D / 16) + (static_cast<long>(hkv) * D) / 8;
  return static_cast<int>(launch_kernel(rope_cache_kernel, dim3(static_cast<unsigned>((per_row * T + 255) / 256)), dim3(256),
                                        0, s, reinterpret_cast<__nv_bfloat16*>(qkv), cos_t, sin_t, cache_rows,
                                        reinterpret_cast<__nv_bfloat16*>(cache), T, W, hq, hkv, D, ld_cache, cache_nrows));
}

bool attn_decode_supported(int Tq, int hq, int hkv, int D) {
  return D == kDecD && hkv >= 1 && hq % hkv == 0 && Tq >= 1 && Tq <= 256;
}

int attn_decode(const void* q, long ldq, const void* k, long ldk, const void* v, long ldv, const void* qtab,
                const void* ktab, void* out, long ldo, int Tq, int Tk, int hq, int hkv, int D, float scale, int max_keys,
                cudaStream_t s) {
  if (!attn_decode_supported(Tq, hq, hkv, D)) return -1;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (ldo % 4)) return -2;
  const int rep = hq / hkv;
  const int warps = rep < kDecMaxWarps ? rep : kDecMaxWarps;
  // fewer than two warps would leave the staging of a block to 32 threads: run at least two
  const int launch_warps = warps < 2 ? 2 : warps;
  const int z = (rep + warps - 1) / warps;
  // one CTA per key block of the longest row, up to the cluster limit (rows with fewer blocks leave CTAs idle)
  const int keys = max_keys > 0 && max_keys < Tk ? max_keys : Tk;
  int splits = (keys + kDecBlock - 1) / kDecBlock;
  splits = splits < 1 ? 1 : (splits > kDecMaxSplits ? kDecMaxSplits : splits);
  static bool attr_set = false;
  const int smem = static_cast<int>(sizeof(DecSmem)) + 16;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set = true;
  }
  return static_cast<int>(launch_kernel_cluster(
      attn_decode_kernel, dim3(static_cast<unsigned>(Tq * splits), static_cast<unsigned>(hkv), static_cast<unsigned>(z)),
      dim3(launch_warps * 32), smem, s, static_cast<unsigned>(splits), reinterpret_cast<const __nv_bfloat16*>(q), ldq,
      reinterpret_cast<const __nv_bfloat16*>(k), ldk, reinterpret_cast<const __nv_bfloat16*>(v), ldv,
      reinterpret_cast<const int4*>(qtab), reinterpret_cast<const int4*>(ktab), reinterpret_cast<__nv_bfloat16*>(out), ldo,
      Tq, Tk, hq, hkv, scale * 1.4426950408889634f, warps, splits));
}

WX_CHK_DEFINE_READER(decode_check_read)

}  // namespace wx
