// Varlen attention on tcgen05 / TMEM / TMA for sm_100a: forward, dQ and dK/dV kernels.
//
// Packed layout: q [Tq, hq*D], k/v [Tk, hkv*D] (row-strided views of one q|k|v buffer are fine).
// A CTA owns 128 consecutive rows of the packed buffer (rows may span several sequences); which
// keys a query may see comes from a per-query table (key range of its sequence, causal limit,
// bidirectional flag), so windows, full images, causal text and the bidirectional action block are
// one code path and tiles never fragment on sequence boundaries.
//
//   forward : S = Q K^T (tcgen05, fp32 in TMEM) -> online softmax in registers (one thread per
//             query row) -> P (bf16) to swizzled smem -> O += P V (tcgen05, accumulator in TMEM).
//   dQ      : per query tile, recompute S and dP = dO V^T, dS -> smem, dQ += dS K.
//   dK/dV   : per key tile and query head, recompute S^T = K Q^T and dP^T = V dO^T,
//             dV += P^T dO, dK += dS^T Q; GQA partials are summed by a small reduce kernel.
// All operand tiles arrive by TMA (no cluster multicast); every wait is bounded.
//
// Reference parity: flash_attn_func / flash_attn_varlen_func as used in
// modeling_qwen2_5_vl.py:208-210 and :1008-1015, and the masked eager path of
// modeling_qwen2_5_vl_act.py:616-637.
#include "attention.h"
#include "ptx.cuh"

#include <math.h>
#include <mutex>

namespace wx {

namespace {

constexpr int AT_THREADS = 128;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

struct AttnArgs {
  CUtensorMap tmQ;    // box {64, 128} (fwd, dq) or {64, 64} (dkdv)
  CUtensorMap tmK;    // box {64, 64} (fwd, dq) or {64, 128} (dkdv)
  CUtensorMap tmV;
  CUtensorMap tmDO;   // like tmQ
  const int4* qtab;   // [Tq] (k_lo, k_hi, k_lim, flag)
  const int4* ktab;   // [Tk] (q_lo, q_hi, first causal viewer row, flag | first viewer row << 1)
  __nv_bfloat16* out;   // fwd: O; dq: dQ
  long ld_out;
  __nv_bfloat16* out2;  // dkdv: dV (bf16, rep == 1)
  long ld_out2;
  float* part_k;        // dkdv: fp32 partials [rep][Tk][hkv*D] (rep > 1)
  float* part_v;
  float* lse;           // [hq, Tq] natural log
  const float* delta;   // [hq, Tq]
  int Tq, Tk, hq, hkv, D;
  float scale;
  int has_bidir;
  int causal_self;
};

struct SmemCtl {
  uint64_t bar[8];
  uint32_t tmem_slot;
  int abort_flag;
  int kmin, kmax;
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Bits c (0..63) with lo <= c <= hi.
__device__ __forceinline__ uint64_t bits_between(int lo, int hi) {
  lo = max(lo, 0);
  hi = min(hi, 63);
  if (hi < lo) return 0ull;
  return (~0ull >> (63 - (hi - lo))) << lo;
}
// Which of the 64 keys starting at kbase a query row may see: its causal interval, plus (for a
// flagged row) the flagged keys of its own sequence. `kflags` has bit c set when key kbase+c is flagged.
__device__ __forceinline__ uint64_t row_key_mask(const int4& qi, int kbase, uint64_t kflags) {
  uint64_t m = bits_between(qi.x - kbase, min(qi.z, qi.y - 1) - kbase);
  if (qi.w != 0) m |= kflags & bits_between(qi.x - kbase, qi.y - 1 - kbase);
  return m;
}
// 64-bit ballot over a shared int[64] of 0/1 flags (all 32 lanes of the warp take part).
__device__ __forceinline__ uint64_t flags_to_mask(const int* flags64) {
  const int lane = threadIdx.x & 31;
  const uint32_t lo = __ballot_sync(0xffffffffu, flags64[lane] != 0);
  const uint32_t hi = __ballot_sync(0xffffffffu, flags64[32 + lane] != 0);
  return (static_cast<uint64_t>(hi) << 32) | lo;
}

__device__ __forceinline__ bool key_allowed(int kk, const int4& qi, int kflag) {
  return kk >= qi.x && kk < qi.y && (kk <= qi.z || (qi.w != 0 && kflag != 0));
}

// ================================================================================ forward
// 160 threads: warps 0..3 own one query row per thread (softmax, O rescale, epilogue); warp 4 is
// the issue warp (one lane drives TMA loads and tcgen05.mma). The two roles talk through mbarriers
// only, so the issuing lane never shares a warp with threads that wait.
// smem: Q 2x[128][64] (32 KB) | stage s in {0,1}: K 2x[64][64] (16 KB) | V 2x[64][64] (16 KB).
// P (16 KB, [128][64] K-major) overwrites the K stage once S has been read.
// Barriers: kv_full[2] (TMA), q_full (TMA), s_bar (QK done), s_free (S copied to registers, 128
// arrivals), p_ready (P in smem and O rescaled, 128 arrivals), pv_bar (PV done).
constexpr int FWD_THREADS = 160;
__global__ void __launch_bounds__(FWD_THREADS, 2)
attn_fwd_kernel(const __grid_constant__ AttnArgs a, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = smem + 32768;  // stage s: K at sKV + s*32768, V at + 16384
  __shared__ SmemCtl ctl;
  __shared__ int s_kflag[2][64];
  uint64_t* kv_full = &ctl.bar[0];  // [2]
  uint64_t* q_full = &ctl.bar[2];
  uint64_t* s_bar = &ctl.bar[3];
  uint64_t* pv_bar = &ctl.bar[4];
  uint64_t* s_free = &ctl.bar[5];
  uint64_t* p_ready = &ctl.bar[6];
  volatile int* abort_flag = &ctl.abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5;
  const bool is_row = warp < 4;
  const int h = blockIdx.y;
  const int g = h / (a.hq / a.hkv);
  const int r0 = blockIdx.x * 128;
  const int row = r0 + tid;
  const bool row_ok = is_row && row < a.Tq;
  const int D = a.D;
  const int nbox = (D + 63) / 64;

  int4 qi = make_int4(0, 0, -1, 0);
  if (row_ok) qi = a.qtab[row];
  // debug build: the row's key range lies inside the key buffer and its causal limit inside that range
  if (row_ok && !WX_CHK(qi.x >= 0 && qi.x <= qi.y && qi.y <= a.Tk && qi.z < qi.y, 3001, qi.x, qi.y)) qi = make_int4(0, 0, -1, 0);
  if (tid == 0) {
    for (int i = 0; i < 5; ++i) mbar_init(&ctl.bar[i], 1);
    mbar_init(s_free, 128);
    mbar_init(p_ready, 128);
    ctl.abort_flag = 0;
    ctl.kmin = 0x7fffffff;
    ctl.kmax = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(&ctl.tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (row_ok) {
    const int upper = qi.w ? qi.y : min(qi.z + 1, qi.y);
    atomicMin(&ctl.kmin, qi.x);
    atomicMax(&ctl.kmax, upper);
  }
  __syncthreads();
  const uint32_t tmem = ctl.tmem_slot;
  const uint32_t tS = tmem;        // 64 columns
  const uint32_t tO = tmem + 128;  // D columns
  const int kmin = ctl.kmin, kmax = ctl.kmax;
  const int nblk = (kmax > kmin) ? (kmax - kmin + 63) / 64 : 0;
  const float scale_log2 = a.scale * LOG2E;
  float m_run = -INFINITY, l_run = 0.f;
  bool ok = nblk > 0;

  if (!is_row) {
    // ------------------------------------------------------------------ issue warp
    if (tid == 128 && nblk > 0) {
      const uint32_t kv_bytes = static_cast<uint32_t>(nbox) * 8192u * 2u;
      const uint32_t idesc_s = make_idesc_bf16(128, 64, false, false);
      const uint32_t idesc_o = make_idesc_bf16(128, D, false, true);
      auto load_kv = [&](int j) {
        const int st = j & 1;
        uint8_t* sK = sKV + st * 32768;
        uint8_t* sV = sK + 16384;
        mbar_arrive_expect_tx(&kv_full[st], kv_bytes);
        for (int b = 0; b < nbox; ++b) {
          tma_load_2d(sK + b * 8192, &a.tmK, &kv_full[st], g * D + b * 64, kmin + j * 64);
          tma_load_2d(sV + b * 8192, &a.tmV, &kv_full[st], g * D + b * 64, kmin + j * 64);
        }
      };
      mbar_arrive_expect_tx(q_full, static_cast<uint32_t>(nbox) * 16384u);
      for (int b = 0; b < nbox; ++b) tma_load_2d(sQ + b * 16384, &a.tmQ, q_full, h * D + b * 64, r0);
      load_kv(0);
      if (nblk > 1) load_kv(1);
      ok = mbar_wait(q_full, 0, abort_flag);
      const uint32_t qa = smem_u32(sQ);
      for (int j = 0; j < nblk && ok; ++j) {
        const int st = j & 1;
        const uint32_t ka = smem_u32(sKV + st * 32768), va = ka + 16384;
        ok = mbar_wait(&kv_full[st], (j >> 1) & 1, abort_flag);
        if (ok && j > 0) ok = mbar_wait(s_free, (j - 1) & 1, abort_flag);  // S(j-1) is in registers
        if (!ok) break;
        tc_fence_after();
        for (int k = 0; k < D / 16; ++k) {
          const uint64_t da = make_smem_desc_sw128(qa + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(ka + (k >> 2) * 8192 + (k & 3) * 32, 16, 1024);
          tc_mma_bf16(tS, da, db, idesc_s, k != 0);
        }
        tc_commit(s_bar);
        // stage (j+1)&1 was last read by PV(j-1): refill it once that is done
        if (j > 0 && j + 1 < nblk) {
          ok = mbar_wait(pv_bar, (j - 1) & 1, abort_flag);
          if (!ok) break;
          load_kv(j + 1);
        }
        ok = mbar_wait(p_ready, j & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint64_t da = make_smem_desc_sw128(ka + k * 32, 16, 1024);          // P lives in the K stage
          const uint64_t db = make_smem_desc_sw128(va + k * 2048, 8192, 1024);
          tc_mma_bf16(tO, da, db, idesc_o, (j | k) != 0);
        }
        tc_commit(pv_bar);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax warps
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
    for (int j = 0; j < nblk; ++j) {
      const int st = j & 1;
      uint8_t* sP = sKV + st * 32768;
      const int kbase = kmin + j * 64;
      if (a.has_bidir && tid < 64) {
        const int kk = kbase + tid;
        s_kflag[st][tid] = (kk < a.Tk) ? (a.ktab[kk].w & 1) : 0;
      }
      if (a.has_bidir) asm volatile("bar.sync 1, 128;" ::: "memory");  // flags visible to the 4 row warps
      if (ok) ok = mbar_wait(s_bar, j & 1, abort_flag);
      tc_fence_after();
      float sc[64];
      {
        uint32_t r[32];
        tmem_ld_32x32(tS + lane_off, r);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; ++c) sc[c] = __uint_as_float(r[c]);
        tmem_ld_32x32(tS + lane_off + 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; ++c) sc[32 + c] = __uint_as_float(r[c]);
      }
      tc_fence_before();
      mbar_arrive(s_free);  // the issue warp may overwrite S with the next block's scores
      // Interior blocks (every key visible to every row of the warp) skip the per-element mask.
      const bool fast = __all_sync(0xffffffffu, kbase >= qi.x && kbase + 63 <= qi.z && kbase + 63 < qi.y);
      float raw_max = -INFINITY;
      if (fast) {
#pragma unroll
        for (int c = 0; c < 64; ++c) raw_max = fmaxf(raw_max, sc[c]);
      } else {
        const uint64_t km = row_key_mask(qi, kbase, a.has_bidir ? flags_to_mask(s_kflag[st]) : 0ull);
        const uint32_t km_lo = static_cast<uint32_t>(km), km_hi = static_cast<uint32_t>(km >> 32);
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          sc[c] = (km_lo & (1u << c)) ? sc[c] : -INFINITY;
          sc[32 + c] = (km_hi & (1u << c)) ? sc[32 + c] : -INFINITY;
          raw_max = fmaxf(raw_max, fmaxf(sc[c], sc[32 + c]));
        }
      }
      const float m_new = fmaxf(m_run, raw_max * scale_log2);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = (m_run == -INFINITY) ? 0.f : ex2_approx(m_run - m_use);
      float psum = 0.f;
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < 64; c += 2) {
        const float p0 = ex2_approx(fmaf(sc[c], scale_log2, -m_use));
        const float p1 = ex2_approx(fmaf(sc[c + 1], scale_log2, -m_use));
        psum += p0 + p1;
        pk[c >> 1] = pack_bf16x2(p0, p1);
      }
      l_run = l_run * alpha + psum;
      const bool changed = m_new > m_run;
      m_run = m_new;
      // PV(j-1) must be done before O is rescaled; P(j) goes to the other stage, which PV(j-2) freed
      if (j > 0) {
        if (ok) ok = mbar_wait(pv_bar, (j - 1) & 1, abort_flag);
        tc_fence_after();
        if (__any_sync(0xffffffffu, changed)) {
          for (int c = 0; c < D; c += 32) {
            uint32_t r[32];
            tmem_ld_32x32(tO + lane_off + c, r);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
            tmem_st_32x32(tO + lane_off + c, r);
          }
          tmem_st_wait();
        }
      }
#pragma unroll
      for (int c16 = 0; c16 < 8; ++c16)
        *reinterpret_cast<uint4*>(sP + sw128_offset(tid, c16)) =
            make_uint4(pk[4 * c16], pk[4 * c16 + 1], pk[4 * c16 + 2], pk[4 * c16 + 3]);
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(p_ready);
    }
    if (ok && nblk > 0) ok = mbar_wait(pv_bar, (nblk - 1) & 1, abort_flag);
    tc_fence_after();
    {
      // TMEM loads are warp-collective: every lane runs them, only the stores are predicated.
      const bool have = __all_sync(0xffffffffu, ok) && nblk > 0;
      const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* orow = a.out + static_cast<long>(row) * a.ld_out + h * D;
      for (int c = 0; c < D; c += 16) {
        uint32_t r[16];
        if (have) {
          tmem_ld_32x16(tO + lane_off + c, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e) r[e] = 0u;
        }
        if (row_ok) {
#pragma unroll
          for (int q2 = 0; q2 < 2; ++q2)
            reinterpret_cast<uint4*>(orow + c)[q2] = make_uint4(
                pack_bf16x2(__uint_as_float(r[8 * q2 + 0]) * inv_l, __uint_as_float(r[8 * q2 + 1]) * inv_l),
                pack_bf16x2(__uint_as_float(r[8 * q2 + 2]) * inv_l, __uint_as_float(r[8 * q2 + 3]) * inv_l),
                pack_bf16x2(__uint_as_float(r[8 * q2 + 4]) * inv_l, __uint_as_float(r[8 * q2 + 5]) * inv_l),
                pack_bf16x2(__uint_as_float(r[8 * q2 + 6]) * inv_l, __uint_as_float(r[8 * q2 + 7]) * inv_l));
        }
      }
      if (row_ok)
        a.lse[static_cast<long>(h) * a.Tq + row] = (have && l_run > 0.f) ? (m_run + log2f(l_run)) * LN2 : -INFINITY;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && ctl.abort_flag) atomicExch(status, 2);
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
}

// ================================================================================ delta
// delta[h, r] = sum_d dO[r, h, d] * O[r, h, d]
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ dO, long ld_do, const __nv_bfloat16* __restrict__ O,
                                  long ld_o, float* __restrict__ delta, int Tq, int hq, int D) {
  const int wid = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= Tq * hq) return;
  const int r = wid / hq, h = wid - r * hq;
  const __nv_bfloat16* a = dO + static_cast<long>(r) * ld_do + h * D;
  const __nv_bfloat16* b = O + static_cast<long>(r) * ld_o + h * D;
  float s = 0.f;
  for (int d = lane * 2; d < D; d += 64) {
    const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(a + d));
    const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(b + d));
    s += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) delta[static_cast<long>(h) * Tq + r] = s;
}

// ================================================================================ dQ
// 160 threads: warps 0..3 own one query row per thread, warp 4 issues TMA and tcgen05.mma.
// smem: Q 2x[128][64] (32 KB) | dO 2x[128][64] (32 KB) | K 2x[64][64] (16 KB) | V 2x[64][64] (16 KB).
// dS ([128][64] K-major, 16 KB) overwrites V once dP has been read.
constexpr int DQ_THREADS = 160;
__global__ void __launch_bounds__(DQ_THREADS, 2)
attn_dq_kernel(const __grid_constant__ AttnArgs a, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sDO = smem + 32768;
  uint8_t* sK = smem + 65536;
  uint8_t* sV = smem + 81920;
  __shared__ SmemCtl ctl;
  __shared__ int s_kflag[2][64];
  uint64_t* kv_full = &ctl.bar[0];
  uint64_t* q_full = &ctl.bar[1];
  uint64_t* s_bar = &ctl.bar[2];
  uint64_t* dq_bar = &ctl.bar[3];
  uint64_t* ds_ready = &ctl.bar[4];
  volatile int* abort_flag = &ctl.abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5;
  const bool is_row = warp < 4;
  const int h = blockIdx.y;
  const int g = h / (a.hq / a.hkv);
  const int r0 = blockIdx.x * 128;
  const int row = r0 + tid;
  const bool row_ok = is_row && row < a.Tq;
  const int D = a.D;
  const int nbox = (D + 63) / 64;

  int4 qi = make_int4(0, 0, -1, 0);
  float lse2 = 0.f, dlt_s = 0.f;
  if (row_ok) {
    qi = a.qtab[row];
    if (!WX_CHK(qi.x >= 0 && qi.x <= qi.y && qi.y <= a.Tk && qi.z < qi.y, 3002, qi.x, qi.y)) qi = make_int4(0, 0, -1, 0);
    lse2 = a.lse[static_cast<long>(h) * a.Tq + row] * LOG2E;
    dlt_s = a.delta[static_cast<long>(h) * a.Tq + row] * a.scale;
  }
  if (tid == 0) {
    for (int i = 0; i < 4; ++i) mbar_init(&ctl.bar[i], 1);
    mbar_init(ds_ready, 128);
    ctl.abort_flag = 0;
    ctl.kmin = 0x7fffffff;
    ctl.kmax = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(&ctl.tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (row_ok) {
    const int upper = qi.w ? qi.y : min(qi.z + 1, qi.y);
    atomicMin(&ctl.kmin, qi.x);
    atomicMax(&ctl.kmax, upper);
  }
  __syncthreads();
  const uint32_t tmem = ctl.tmem_slot;
  const uint32_t tS = tmem, tDP = tmem + 64, tDQ = tmem + 128;
  const int kmin = ctl.kmin, kmax = ctl.kmax;
  const int nblk = (kmax > kmin) ? (kmax - kmin + 63) / 64 : 0;
  const float scale_log2 = a.scale * LOG2E;
  bool ok = nblk > 0;

  if (!is_row) {
    if (tid == 128 && nblk > 0) {
      const uint32_t kv_bytes = static_cast<uint32_t>(nbox) * 8192u * 2u;
      const uint32_t idesc_s = make_idesc_bf16(128, 64, false, false);
      const uint32_t idesc_dq = make_idesc_bf16(128, D, false, true);
      auto load_kv = [&](int j) {
        mbar_arrive_expect_tx(kv_full, kv_bytes);
        for (int b = 0; b < nbox; ++b) {
          tma_load_2d(sK + b * 8192, &a.tmK, kv_full, g * D + b * 64, kmin + j * 64);
          tma_load_2d(sV + b * 8192, &a.tmV, kv_full, g * D + b * 64, kmin + j * 64);
        }
      };
      mbar_arrive_expect_tx(q_full, static_cast<uint32_t>(nbox) * 16384u * 2u);
      for (int b = 0; b < nbox; ++b) {
        tma_load_2d(sQ + b * 16384, &a.tmQ, q_full, h * D + b * 64, r0);
        tma_load_2d(sDO + b * 16384, &a.tmDO, q_full, h * D + b * 64, r0);
      }
      load_kv(0);
      ok = mbar_wait(q_full, 0, abort_flag);
      const uint32_t qa = smem_u32(sQ), da_ = smem_u32(sDO), ka = smem_u32(sK), va = smem_u32(sV);
      for (int j = 0; j < nblk && ok; ++j) {
        ok = mbar_wait(kv_full, j & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t ao = (k >> 2) * 16384 + (k & 3) * 32, bo = (k >> 2) * 8192 + (k & 3) * 32;
          tc_mma_bf16(tS, make_smem_desc_sw128(qa + ao, 16, 1024), make_smem_desc_sw128(ka + bo, 16, 1024), idesc_s, k != 0);
        }
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t ao = (k >> 2) * 16384 + (k & 3) * 32, bo = (k >> 2) * 8192 + (k & 3) * 32;
          tc_mma_bf16(tDP, make_smem_desc_sw128(da_ + ao, 16, 1024), make_smem_desc_sw128(va + bo, 16, 1024), idesc_s, k != 0);
        }
        tc_commit(s_bar);
        ok = mbar_wait(ds_ready, j & 1, abort_flag);  // dS is in smem (over V)
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 4; ++k)
          tc_mma_bf16(tDQ, make_smem_desc_sw128(va + k * 32, 16, 1024), make_smem_desc_sw128(ka + k * 2048, 8192, 1024),
                      idesc_dq, (j | k) != 0);
        tc_commit(dq_bar);
        if (j + 1 < nblk) {  // K and dS are read by the MMA just issued: refill when it is done
          ok = mbar_wait(dq_bar, j & 1, abort_flag);
          if (!ok) break;
          load_kv(j + 1);
        }
      }
    }
  } else {
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
    for (int j = 0; j < nblk; ++j) {
      const int st = j & 1;
      const int kbase = kmin + j * 64;
      if (a.has_bidir) {
        if (tid < 64) {
          const int kk = kbase + tid;
          s_kflag[st][tid] = (kk < a.Tk) ? (a.ktab[kk].w & 1) : 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      if (ok) ok = mbar_wait(s_bar, j & 1, abort_flag);
      tc_fence_after();
      const bool fast = __all_sync(0xffffffffu, kbase >= qi.x && kbase + 63 <= qi.z && kbase + 63 < qi.y);
      uint64_t km = ~0ull;
      if (!fast) km = row_key_mask(qi, kbase, a.has_bidir ? flags_to_mask(s_kflag[st]) : 0ull);
      uint32_t pk[32];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t rs[32], rp[32];
        tmem_ld_32x32(tS + lane_off + half * 32, rs);
        tmem_ld_32x32(tDP + lane_off + half * 32, rp);
        tmem_ld_wait();
        const uint32_t kmh = static_cast<uint32_t>(km >> (32 * half));
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          float p0 = ex2_approx(fmaf(__uint_as_float(rs[c]), scale_log2, -lse2));
          float p1 = ex2_approx(fmaf(__uint_as_float(rs[c + 1]), scale_log2, -lse2));
          if (!fast) {
            p0 = (kmh & (1u << c)) ? p0 : 0.f;
            p1 = (kmh & (2u << c)) ? p1 : 0.f;
          }
          pk[(half * 32 + c) >> 1] = pack_bf16x2(p0 * fmaf(__uint_as_float(rp[c]), a.scale, -dlt_s),
                                                 p1 * fmaf(__uint_as_float(rp[c + 1]), a.scale, -dlt_s));
        }
      }
#pragma unroll
      for (int c16 = 0; c16 < 8; ++c16)
        *reinterpret_cast<uint4*>(sV + sw128_offset(tid, c16)) =
            make_uint4(pk[4 * c16], pk[4 * c16 + 1], pk[4 * c16 + 2], pk[4 * c16 + 3]);
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(ds_ready);
    }
    if (ok && nblk > 0) ok = mbar_wait(dq_bar, (nblk - 1) & 1, abort_flag);
    tc_fence_after();
    {
      const bool have = __all_sync(0xffffffffu, ok) && nblk > 0;
      __nv_bfloat16* orow = a.out + static_cast<long>(row) * a.ld_out + h * D;
      for (int c = 0; c < D; c += 16) {
        uint32_t r[16];
        if (have) {
          tmem_ld_32x16(tDQ + lane_off + c, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e) r[e] = 0u;
        }
        if (row_ok) {
#pragma unroll
          for (int q2 = 0; q2 < 2; ++q2)
            reinterpret_cast<uint4*>(orow + c)[q2] =
                make_uint4(pack_bf16x2(__uint_as_float(r[8 * q2 + 0]), __uint_as_float(r[8 * q2 + 1])),
                           pack_bf16x2(__uint_as_float(r[8 * q2 + 2]), __uint_as_float(r[8 * q2 + 3])),
                           pack_bf16x2(__uint_as_float(r[8 * q2 + 4]), __uint_as_float(r[8 * q2 + 5])),
                           pack_bf16x2(__uint_as_float(r[8 * q2 + 6]), __uint_as_float(r[8 * q2 + 7])));
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && ctl.abort_flag) atomicExch(status, 3);
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
}

// ================================================================================ dK / dV
// One CTA: 128 keys of kv head g, one query head h. 160 threads: warps 0..3 own one key row per
// thread, warp 4 issues TMA and tcgen05.mma. smem: K 2x[128][64] (32 KB) | V (32 KB) | stage s in
// {0,1}: Q_i 2x[64][64] (16 KB) + dO_i (16 KB) | P^T [128][64] (16 KB) | dS^T (16 KB).
// Which query columns a key row may be seen by is an interval of rows (from the first causal
// viewer to the end of the sequence) plus, for a flagged key, the flagged queries of the sequence:
// one 64-bit mask per thread and block, no per-element table look-ups.
constexpr int DKDV_THREADS = 160;
__global__ void __launch_bounds__(DKDV_THREADS, 1)
attn_dkdv_kernel(const __grid_constant__ AttnArgs a, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + 32768;
  uint8_t* sQD = smem + 65536;         // stage s: Q at + s*32768, dO at + 16384
  uint8_t* sPT = smem + 65536 + 65536;
  uint8_t* sDST = sPT + 16384;
  __shared__ SmemCtl ctl;
  __shared__ __align__(16) float2 s_ld[2][64];  // (lse * log2e, delta * scale) per query column
  __shared__ int s_qflag[2][64];
  uint64_t* qd_full = &ctl.bar[0];  // [2]
  uint64_t* kv_full = &ctl.bar[2];
  uint64_t* s_bar = &ctl.bar[3];
  uint64_t* acc_bar = &ctl.bar[4];
  uint64_t* sp_free = &ctl.bar[5];
  uint64_t* pt_ready = &ctl.bar[6];
  volatile int* abort_flag = &ctl.abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5;
  const bool is_row = warp < 4;
  const int rep = a.hq / a.hkv;
  const int g = blockIdx.y / rep;
  const int hsub = blockIdx.y - g * rep;
  const int h = g * rep + hsub;
  const int c0 = blockIdx.x * 128;
  const int key = c0 + tid;
  const bool key_ok = is_row && key < a.Tk;
  const int D = a.D;
  const int nbox = (D + 63) / 64;

  int4 ki = make_int4(0, 0, 0x7fffffff, 0);  // (q_lo, q_hi, first causal viewer, flag | first viewer << 1)
  if (key_ok) ki = a.ktab[key];
  // debug build: the key's query range lies inside the query buffer
  if (key_ok && !WX_CHK(ki.x >= 0 && ki.x <= ki.y && ki.y <= a.Tq, 3003, ki.x, ki.y)) ki = make_int4(0, 0, 0x7fffffff, 0);
  const int kflag = ki.w & 1;
  if (tid == 0) {
    for (int i = 0; i < 5; ++i) mbar_init(&ctl.bar[i], 1);
    mbar_init(sp_free, 128);
    mbar_init(pt_ready, 128);
    ctl.abort_flag = 0;
    ctl.kmin = 0x7fffffff;
    ctl.kmax = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(&ctl.tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (key_ok) {
    atomicMin(&ctl.kmin, ki.w >> 1);  // first query row that can see this key
    atomicMax(&ctl.kmax, ki.y);
  }
  __syncthreads();
  const uint32_t tmem = ctl.tmem_slot;
  const uint32_t tS = tmem, tDP = tmem + 64, tDV = tmem + 128, tDK = tmem + 256;
  const int qmin = ctl.kmin;
  const int qmax = ctl.kmax;
  const int nblk = (qmax > qmin) ? (qmax - qmin + 63) / 64 : 0;
  const float scale_log2 = a.scale * LOG2E;
  bool ok = nblk > 0;

  if (!is_row) {
    if (tid == 128 && nblk > 0) {
      const uint32_t qd_bytes = static_cast<uint32_t>(nbox) * 8192u * 2u;
      const uint32_t idesc_s = make_idesc_bf16(128, 64, false, false);
      const uint32_t idesc_acc = make_idesc_bf16(128, D, false, true);
      auto load_qd = [&](int i) {
        const int st = i & 1;
        uint8_t* q = sQD + st * 32768;
        uint8_t* d = q + 16384;
        mbar_arrive_expect_tx(&qd_full[st], qd_bytes);
        for (int b = 0; b < nbox; ++b) {
          tma_load_2d(q + b * 8192, &a.tmQ, &qd_full[st], h * D + b * 64, qmin + i * 64);
          tma_load_2d(d + b * 8192, &a.tmDO, &qd_full[st], h * D + b * 64, qmin + i * 64);
        }
      };
      mbar_arrive_expect_tx(kv_full, static_cast<uint32_t>(nbox) * 16384u * 2u);
      for (int b = 0; b < nbox; ++b) {
        tma_load_2d(sK + b * 16384, &a.tmK, kv_full, g * D + b * 64, c0);
        tma_load_2d(sV + b * 16384, &a.tmV, kv_full, g * D + b * 64, c0);
      }
      load_qd(0);
      if (nblk > 1) load_qd(1);
      ok = mbar_wait(kv_full, 0, abort_flag);
      const uint32_t ka = smem_u32(sK), va = smem_u32(sV), pa = smem_u32(sPT), sa = smem_u32(sDST);
      for (int i = 0; i < nblk && ok; ++i) {
        const int st = i & 1;
        const uint32_t qa = smem_u32(sQD + st * 32768), da_ = qa + 16384;
        ok = mbar_wait(&qd_full[st], (i >> 1) & 1, abort_flag);
        if (ok && i > 0) ok = mbar_wait(sp_free, (i - 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t ao = (k >> 2) * 16384 + (k & 3) * 32, bo = (k >> 2) * 8192 + (k & 3) * 32;
          tc_mma_bf16(tS, make_smem_desc_sw128(ka + ao, 16, 1024), make_smem_desc_sw128(qa + bo, 16, 1024), idesc_s, k != 0);
        }
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t ao = (k >> 2) * 16384 + (k & 3) * 32, bo = (k >> 2) * 8192 + (k & 3) * 32;
          tc_mma_bf16(tDP, make_smem_desc_sw128(va + ao, 16, 1024), make_smem_desc_sw128(da_ + bo, 16, 1024), idesc_s, k != 0);
        }
        tc_commit(s_bar);
        if (i > 0 && i + 1 < nblk) {  // stage (i+1)&1 was read by the accumulating MMAs of block i-1
          ok = mbar_wait(acc_bar, (i - 1) & 1, abort_flag);
          if (!ok) break;
          load_qd(i + 1);
        }
        ok = mbar_wait(pt_ready, i & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 4; ++k)
          tc_mma_bf16(tDV, make_smem_desc_sw128(pa + k * 32, 16, 1024), make_smem_desc_sw128(da_ + k * 2048, 8192, 1024),
                      idesc_acc, (i | k) != 0);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          tc_mma_bf16(tDK, make_smem_desc_sw128(sa + k * 32, 16, 1024), make_smem_desc_sw128(qa + k * 2048, 8192, 1024),
                      idesc_acc, (i | k) != 0);
        tc_commit(acc_bar);
      }
    }
  } else {
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
    for (int i = 0; i < nblk; ++i) {
      const int st = i & 1;
      const int qbase = qmin + i * 64;
      if (tid < 64) {
        const int qr = qbase + tid;
        float2 ld = make_float2(0.f, 0.f);
        int fq = 0;
        if (qr < a.Tq) {
          ld.x = a.lse[static_cast<long>(h) * a.Tq + qr] * LOG2E;
          ld.y = a.delta[static_cast<long>(h) * a.Tq + qr] * a.scale;
          fq = a.has_bidir ? a.qtab[qr].w : 0;
        }
        s_ld[st][tid] = ld;
        s_qflag[st][tid] = fq;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");  // per-query values visible to the 4 row warps
      uint64_t qm = bits_between(ki.z - qbase, ki.y - 1 - qbase);
      if (a.has_bidir) {
        const uint64_t qfm = flags_to_mask(s_qflag[st]);
        if (kflag) qm |= qfm & bits_between(ki.x - qbase, ki.y - 1 - qbase);
      }
      if (!key_ok) qm = 0ull;
      const bool fast = __all_sync(0xffffffffu, qm == ~0ull);
      if (ok) ok = mbar_wait(s_bar, i & 1, abort_flag);
      tc_fence_after();
      uint32_t pp[32], pd[32];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t rs[32], rp[32];
        tmem_ld_32x32(tS + lane_off + half * 32, rs);
        tmem_ld_32x32(tDP + lane_off + half * 32, rp);
        tmem_ld_wait();
        const uint32_t qmh = static_cast<uint32_t>(qm >> (32 * half));
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          const float4 l2 = *reinterpret_cast<const float4*>(&s_ld[st][half * 32 + c]);
          float p0 = ex2_approx(fmaf(__uint_as_float(rs[c]), scale_log2, -l2.x));
          float p1 = ex2_approx(fmaf(__uint_as_float(rs[c + 1]), scale_log2, -l2.z));
          if (!fast) {
            p0 = (qmh & (1u << c)) ? p0 : 0.f;
            p1 = (qmh & (2u << c)) ? p1 : 0.f;
          }
          pp[(half * 32 + c) >> 1] = pack_bf16x2(p0, p1);
          pd[(half * 32 + c) >> 1] = pack_bf16x2(p0 * fmaf(__uint_as_float(rp[c]), a.scale, -l2.y),
                                                 p1 * fmaf(__uint_as_float(rp[c + 1]), a.scale, -l2.w));
        }
      }
      tc_fence_before();
      mbar_arrive(sp_free);  // S^T / dP^T are in registers: the next block's scores may overwrite them
      // the accumulating MMAs of the previous block read sPT / sDST
      if (i > 0) {
        if (ok) ok = mbar_wait(acc_bar, (i - 1) & 1, abort_flag);
      }
#pragma unroll
      for (int c16 = 0; c16 < 8; ++c16) {
        *reinterpret_cast<uint4*>(sPT + sw128_offset(tid, c16)) =
            make_uint4(pp[4 * c16], pp[4 * c16 + 1], pp[4 * c16 + 2], pp[4 * c16 + 3]);
        *reinterpret_cast<uint4*>(sDST + sw128_offset(tid, c16)) =
            make_uint4(pd[4 * c16], pd[4 * c16 + 1], pd[4 * c16 + 2], pd[4 * c16 + 3]);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(pt_ready);
    }
    if (ok && nblk > 0) ok = mbar_wait(acc_bar, (nblk - 1) & 1, abort_flag);
    tc_fence_after();
    {
      const bool have = __all_sync(0xffffffffu, ok) && nblk > 0;
      const long W = static_cast<long>(a.hkv) * D;
      __nv_bfloat16* krow = a.out + static_cast<long>(key) * a.ld_out + g * D;
      __nv_bfloat16* vrow = a.out2 + static_cast<long>(key) * a.ld_out2 + g * D;
      float* pkrow = a.part_k + (static_cast<long>(hsub) * a.Tk + key) * W + g * D;
      float* pvrow = a.part_v + (static_cast<long>(hsub) * a.Tk + key) * W + g * D;
      for (int c = 0; c < D; c += 16) {
        uint32_t rk[16], rv[16];
        if (have) {
          tmem_ld_32x16(tDK + lane_off + c, rk);
          tmem_ld_32x16(tDV + lane_off + c, rv);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e) rk[e] = rv[e] = 0u;
        }
        if (!key_ok) continue;
        if (rep == 1) {
#pragma unroll
          for (int q2 = 0; q2 < 2; ++q2) {
            reinterpret_cast<uint4*>(krow + c)[q2] = make_uint4(
                pack_bf16x2(__uint_as_float(rk[8 * q2 + 0]), __uint_as_float(rk[8 * q2 + 1])),
                pack_bf16x2(__uint_as_float(rk[8 * q2 + 2]), __uint_as_float(rk[8 * q2 + 3])),
                pack_bf16x2(__uint_as_float(rk[8 * q2 + 4]), __uint_as_float(rk[8 * q2 + 5])),
                pack_bf16x2(__uint_as_float(rk[8 * q2 + 6]), __uint_as_float(rk[8 * q2 + 7])));
            reinterpret_cast<uint4*>(vrow + c)[q2] = make_uint4(
                pack_bf16x2(__uint_as_float(rv[8 * q2 + 0]), __uint_as_float(rv[8 * q2 + 1])),
                pack_bf16x2(__uint_as_float(rv[8 * q2 + 2]), __uint_as_float(rv[8 * q2 + 3])),
                pack_bf16x2(__uint_as_float(rv[8 * q2 + 4]), __uint_as_float(rv[8 * q2 + 5])),
                pack_bf16x2(__uint_as_float(rv[8 * q2 + 6]), __uint_as_float(rv[8 * q2 + 7])));
          }
        } else {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            reinterpret_cast<float4*>(pkrow + c)[q4] =
                make_float4(__uint_as_float(rk[4 * q4]), __uint_as_float(rk[4 * q4 + 1]), __uint_as_float(rk[4 * q4 + 2]),
                            __uint_as_float(rk[4 * q4 + 3]));
            reinterpret_cast<float4*>(pvrow + c)[q4] =
                make_float4(__uint_as_float(rv[4 * q4]), __uint_as_float(rv[4 * q4 + 1]), __uint_as_float(rv[4 * q4 + 2]),
                            __uint_as_float(rv[4 * q4 + 3]));
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && ctl.abort_flag) atomicExch(status, 4);
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// sum of `rep` fp32 partials -> bf16 (row pitch ld_out)
__global__ void attn_reduce_partials_kernel(const float* __restrict__ part, __nv_bfloat16* __restrict__ out, long ld_out,
                                            int rep, long rows, int W) {
  const long idx = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long total = rows * (W / 4);
  if (idx >= total) return;
  const long r = idx / (W / 4);
  const int c = static_cast<int>(idx - r * (W / 4)) * 4;
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int p = 0; p < rep; ++p) {
    const float4 v = *reinterpret_cast<const float4*>(part + (static_cast<long>(p) * rows + r) * W + c);
    s.x += v.x;
    s.y += v.y;
    s.z += v.z;
    s.w += v.w;
  }
  __nv_bfloat16* o = out + r * ld_out + c;
  *reinterpret_cast<__nv_bfloat162*>(o) = __floats2bfloat162_rn(s.x, s.y);
  *reinterpret_cast<__nv_bfloat162*>(o + 2) = __floats2bfloat162_rn(s.z, s.w);
}

// --------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}
bool tmap2d(CUtensorMap* out, const void* ptr, uint64_t width, uint64_t rows, uint64_t pitch, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  // the encode call is a driver call: make sure this thread has the primary context bound
  thread_local bool bound = false;
  if (!bound) {
    cudaFree(nullptr);
    bound = true;
  }
  cuuint64_t dims[2] = {width, rows};
  cuuint64_t strides[1] = {pitch * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t es[2] = {1, 1};
  return fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

constexpr int FWD_SMEM = 32768 + 65536 + 1024;
constexpr int DQ_SMEM = 98304 + 1024;
constexpr int DKDV_SMEM = 65536 + 65536 + 32768 + 1024;

bool shape_ok(const AttnShape& s) {
  return s.D % 16 == 0 && s.D >= 16 && s.D <= 128 && s.hq % s.hkv == 0 && s.ld_q % 8 == 0 && s.ld_k % 8 == 0 &&
         s.ld_v % 8 == 0 && (s.hq * s.D) % 8 == 0;
}

}  // namespace

WX_CHK_DEFINE_READER(attn_check_read)

int attn_fwd(const AttnShape& s, const void* q, const void* k, const void* v, const void* qtab, const void* ktab,
             void* out, long ld_out, float* lse, cudaStream_t stream, int* status) {
  if (!shape_ok(s)) return -1;
  if (s.Tq == 0) return 0;
  AttnArgs a{};
  if (!tmap2d(&a.tmQ, q, static_cast<uint64_t>(s.hq) * s.D, s.Tq, s.ld_q, 128)) return -2;
  if (!tmap2d(&a.tmK, k, static_cast<uint64_t>(s.hkv) * s.D, s.Tk, s.ld_k, 64)) return -2;
  if (!tmap2d(&a.tmV, v, static_cast<uint64_t>(s.hkv) * s.D, s.Tk, s.ld_v, 64)) return -2;
  a.qtab = reinterpret_cast<const int4*>(qtab);
  a.ktab = reinterpret_cast<const int4*>(ktab);
  a.out = reinterpret_cast<__nv_bfloat16*>(out);
  a.ld_out = ld_out;
  a.lse = lse;
  a.Tq = s.Tq; a.Tk = s.Tk; a.hq = s.hq; a.hkv = s.hkv; a.D = s.D;
  a.scale = s.scale;
  a.has_bidir = s.has_bidir;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr = true;
  }
  dim3 grid((s.Tq + 127) / 128, s.hq);
  attn_fwd_kernel<<<grid, FWD_THREADS, FWD_SMEM, stream>>>(a, status);
  return static_cast<int>(cudaGetLastError());
}

int attn_bwd(const AttnShape& s, const void* q, const void* k, const void* v, const void* out, long ld_o,
             const void* dout, long ld_do, const float* lse, const void* qtab, const void* ktab, float* delta,
             void* dq, long ld_dq, void* dk, long ld_dk, void* dv, long ld_dv, float* part_k, float* part_v,
             cudaStream_t stream, int* status) {
  if (!shape_ok(s) || ld_do % 8 != 0) return -1;
  if (s.Tq == 0 || s.Tk == 0) return 0;
  {
    const long warps = static_cast<long>(s.Tq) * s.hq;
    attn_delta_kernel<<<static_cast<unsigned>((warps * 32 + 255) / 256), 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(dout), ld_do, reinterpret_cast<const __nv_bfloat16*>(out), ld_o, delta,
        s.Tq, s.hq, s.D);
  }
  const int rep = s.hq / s.hkv;
  AttnArgs a{};
  a.qtab = reinterpret_cast<const int4*>(qtab);
  a.ktab = reinterpret_cast<const int4*>(ktab);
  a.lse = const_cast<float*>(lse);
  a.delta = delta;
  a.Tq = s.Tq; a.Tk = s.Tk; a.hq = s.hq; a.hkv = s.hkv; a.D = s.D;
  a.scale = s.scale;
  a.has_bidir = s.has_bidir;
  a.causal_self = s.causal_self;
  // ---- dQ
  if (!tmap2d(&a.tmQ, q, static_cast<uint64_t>(s.hq) * s.D, s.Tq, s.ld_q, 128)) return -2;
  if (!tmap2d(&a.tmDO, dout, static_cast<uint64_t>(s.hq) * s.D, s.Tq, ld_do, 128)) return -2;
  if (!tmap2d(&a.tmK, k, static_cast<uint64_t>(s.hkv) * s.D, s.Tk, s.ld_k, 64)) return -2;
  if (!tmap2d(&a.tmV, v, static_cast<uint64_t>(s.hkv) * s.D, s.Tk, s.ld_v, 64)) return -2;
  a.out = reinterpret_cast<__nv_bfloat16*>(dq);
  a.ld_out = ld_dq;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(attn_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DQ_SMEM);
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaFuncSetAttribute(attn_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DKDV_SMEM);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr = true;
  }
  attn_dq_kernel<<<dim3((s.Tq + 127) / 128, s.hq), DQ_THREADS, DQ_SMEM, stream>>>(a, status);
  // ---- dK / dV
  if (!tmap2d(&a.tmQ, q, static_cast<uint64_t>(s.hq) * s.D, s.Tq, s.ld_q, 64)) return -2;
  if (!tmap2d(&a.tmDO, dout, static_cast<uint64_t>(s.hq) * s.D, s.Tq, ld_do, 64)) return -2;
  if (!tmap2d(&a.tmK, k, static_cast<uint64_t>(s.hkv) * s.D, s.Tk, s.ld_k, 128)) return -2;
  if (!tmap2d(&a.tmV, v, static_cast<uint64_t>(s.hkv) * s.D, s.Tk, s.ld_v, 128)) return -2;
  a.out = reinterpret_cast<__nv_bfloat16*>(dk);
  a.ld_out = ld_dk;
  a.out2 = reinterpret_cast<__nv_bfloat16*>(dv);
  a.ld_out2 = ld_dv;
  a.part_k = part_k;
  a.part_v = part_v;
  if (rep > 1 && (part_k == nullptr || part_v == nullptr)) return -3;
  attn_dkdv_kernel<<<dim3((s.Tk + 127) / 128, s.hq), DKDV_THREADS, DKDV_SMEM, stream>>>(a, status);
  if (rep > 1) {
    const int W = s.hkv * s.D;
    const long total = static_cast<long>(s.Tk) * (W / 4);
    attn_reduce_partials_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
        part_k, reinterpret_cast<__nv_bfloat16*>(dk), ld_dk, rep, s.Tk, W);
    attn_reduce_partials_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
        part_v, reinterpret_cast<__nv_bfloat16*>(dv), ld_dv, rep, s.Tk, W);
  }
  return static_cast<int>(cudaGetLastError());
}

}  // namespace wx
