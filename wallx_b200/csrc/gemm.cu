// tcgen05 / TMEM / TMA GEMM core for sm_100a.
//
// Persistent, warp-specialised kernel, one CTA per SM:
//   warp 0      TMA producer   (one lane): global -> 128B-swizzled shared-memory stages
//   warp 1      MMA issuer     (one lane): tcgen05.mma 128 x BN x 16 per instruction, fp32
//                                          accumulators in tensor memory, double buffered
//   warps 2..9  epilogue       (256 thr):  tcgen05.ld -> bias / GELU / SwiGLU / residual /   (two warps per
//                                          TMEM lane quarter, half of the tile's columns each)
//                                          row scatter / accumulate -> global
// The producer, the issuer and the epilogue are decoupled by mbarriers, so the epilogue of tile
// i overlaps the main loop of tile i+1. All four operand layouts are handled with UMMA
// descriptors (K-major and MN-major, 128-byte swizzle), so forward, dgrad and wgrad need no
// transposed copies. No load uses cluster multicast.
//
// Reference parity: csrc/dual_asym_grouped_gemm.cu:49-136 (two problems, four layouts) and the
// cuBLAS calls behind every nn.Linear in wall_x/model.
#include "gemm.h"
#include "devinfo.h"
#include "launch.h"
#include "ptx.cuh"

#include <cstdlib>
#include <mutex>

namespace wx {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kThreads = 320;  // TMA warp, MMA warp, 8 epilogue warps (two per TMEM lane quarter)
constexpr int kEpiWarps = 8;
constexpr int kEpiWarp0 = 2;

struct Problem {
  CUtensorMap tmA;
  CUtensorMap tmB;
  void* D;
  void* D2;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  const int* row_map;
  const int* dyn;
  long ldd, ldd2, ldr, d_rows;
  int M, N, K, m0, k0, flags;
};

// Device view of a fused weight gather (see AgInfo). The weight is one run of `total_bytes`
// bytes cut into chunks of `chunk_bytes` (a divisor of both the shard size and the 256-row tile
// size, so a chunk never straddles a rank or a tile).
struct AgDev {
  const uint8_t* peer[8];
  uint8_t* staging;
  int* flags;
  long shard_bytes, tile_bytes, total_bytes;
  int chunk_bytes, n_pullers, target, rot, ntiles;
  int cpt, last_chunks, cps;  // chunks per full tile, in the last tile, per shard
};

struct GemmArgs {
  Problem p[2];
  int nprob;
  int raster_group;  // 0: default
  AgDev ag[2];  // used by the AG instantiations only
  // AG instantiations: 1 = ag[i] is the B operand of problem i and the producers wait for its tiles (fused gather);
  // 0 = the copy CTAs fetch `n_ag` weights for LATER launches while this launch multiplies operands that are already
  // in place (prefetch: nothing in this launch waits for them)
  int ag_wait;
  int n_ag;
};

constexpr int kAgRing = 12;          // 16 KB buffers in the (otherwise unused) stage area of a puller CTA
constexpr int kAgChunkMax = 16384;
constexpr int kAgDepth = kAgRing - 2;  // loads in flight
constexpr int kAgLag = 3;               // store groups that may still be in flight behind a published tile
constexpr int kAgPend = 8;              // tiles waiting for their stores' completion (power of two)

template <int BN>
struct Cfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : (BN == 128) ? 6 : 8;
  static constexpr int TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
};

constexpr int kRasterGroup = 8;

struct TileInfo {
  int prob, mt, nt;
};

struct Dims {
  int M[2], K[2], m0[2], k0[2], tiles_m[2], tiles_n[2], tiles[2];
  int group;  // row tiles per raster band
};

template <int BN, int TM = BM>
__device__ __forceinline__ void load_dims(const GemmArgs& args, Dims& d) {
  d.group = args.raster_group > 0 ? args.raster_group : kRasterGroup;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (i < args.nprob) {
      const Problem& p = args.p[i];
      int M = p.M, K = p.K, m0 = p.m0, k0 = p.k0;
      if (p.dyn != nullptr) {  // negative entries keep the static value
        const int d0 = p.dyn[0], d1 = p.dyn[1], d2 = p.dyn[2], d3 = p.dyn[3];
        if (d0 >= 0) m0 = d0;
        if (d1 >= 0) M = min(d1, p.M);
        if (d2 >= 0) k0 = d2;
        if (d3 >= 0) K = d3;
      }
      d.M[i] = M;
      d.K[i] = K;
      d.m0[i] = m0;
      d.k0[i] = k0;
      d.tiles_m[i] = (M + TM - 1) / TM;
      d.tiles_n[i] = (p.N + BN - 1) / BN;
      d.tiles[i] = (K > 0) ? d.tiles_m[i] * d.tiles_n[i] : 0;
    } else {
      d.M[i] = d.K[i] = d.m0[i] = d.k0[i] = d.tiles_m[i] = d.tiles_n[i] = d.tiles[i] = 0;
    }
  }
}

__device__ __forceinline__ TileInfo decode_tile(const Dims& d, int t, bool gathered = false, int rot0 = 0, int rot1 = 0) {
  TileInfo ti;
  ti.prob = 0;
  if (t >= d.tiles[0]) {
    ti.prob = 1;
    t -= d.tiles[0];
  }
  // Grouped raster: tiles are walked in bands of kRasterGroup row tiles, column by column inside a
  // band, so that the CTAs running at the same time cover about 8 row tiles x 8..18 column tiles.
  // Every A tile is then shared by the CTAs of its row and every B tile by the 8 CTAs of its column
  // through L2, instead of one operand being streamed from DRAM once per tile of the other.
  // (With gathered weights the column order is the arrival order: one band, rows fastest.)
  const int tm = d.tiles_m[ti.prob];
  if (gathered) {
    ti.nt = t / tm;
    ti.mt = t - ti.nt * tm;
  } else {
    const int tn = d.tiles_n[ti.prob];
    const int G = d.group;
    const int per_band = G * tn;
    const int band = t / per_band;
    const int r = t - band * per_band;
    const int m_first = band * G;
    const int gm = min(G, tm - m_first);
    ti.nt = r / gm;
    ti.mt = m_first + (r - ti.nt * gm);
  }
  const int rot = gathered ? (ti.prob ? rot1 : rot0) : 0;
  if (rot) {  // gathered weights: start with the tiles this rank owns
    ti.nt += rot;
    const int tn = d.tiles_n[ti.prob];
    if (ti.nt >= tn) ti.nt -= tn;
  }
  return ti;
}

__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }

// Bias / activation / residual / accumulate and the store of 32 consecutive columns [n0, n0 + 32) of destination row
// `drow`: `v` holds the fp32 accumulators (ignored for `zero_row`, which stores zeros: padding rows of a segment).
__device__ __forceinline__ void epilogue_chunk(const Problem& p, float (&v)[32], long drow, int n0, bool zero_row) {
  const int flags = p.flags;
  const bool swiglu = (flags & GEMM_ACT_SWIGLU) != 0;
  const bool out_fp32 = (flags & GEMM_OUT_FP32) != 0;
  const bool accum = (flags & GEMM_ACCUMULATE) != 0 && !zero_row;
  const int nvalid = min(32, p.N - n0);
  if (p.bias != nullptr && !zero_row) {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < nvalid) v[j] += __bfloat162float(p.bias[n0 + j]);
  }
  if (flags & GEMM_SWIGLU_BWD) {
    // v = dL/dh for channels [n0, n0 + 32): two 32-column blocks [16 gate | 16 up] of the saved raw values
    const uint4* gsrc =
        reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.D2) + drow * p.ldd2 + 2 * n0);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.D) + drow * p.ldd + 2 * n0);
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
      uint4 raw[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) raw[q] = zero_row ? make_uint4(0u, 0u, 0u, 0u) : gsrc[4 * blk + q];
      const __nv_bfloat162* gb = reinterpret_cast<const __nv_bfloat162*>(&raw[0]);  // 16 gate values
      const __nv_bfloat162* ub = reinterpret_cast<const __nv_bfloat162*>(&raw[2]);  // 16 up values
      uint32_t og[8], ou[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float2 g2 = __bfloat1622float2(gb[e]);
        const float2 u2 = __bfloat1622float2(ub[e]);
        const float d0 = v[16 * blk + 2 * e], d1 = v[16 * blk + 2 * e + 1];
        const float s0 = 1.0f / (1.0f + __expf(-g2.x)), s1 = 1.0f / (1.0f + __expf(-g2.y));
        og[e] = pack_bf16x2(d0 * u2.x * s0 * (1.0f + g2.x * (1.0f - s0)), d1 * u2.y * s1 * (1.0f + g2.y * (1.0f - s1)));
        ou[e] = pack_bf16x2(d0 * g2.x * s0, d1 * g2.y * s1);
      }
      dst[4 * blk + 0] = make_uint4(og[0], og[1], og[2], og[3]);
      dst[4 * blk + 1] = make_uint4(og[4], og[5], og[6], og[7]);
      dst[4 * blk + 2] = make_uint4(ou[0], ou[1], ou[2], ou[3]);
      dst[4 * blk + 3] = make_uint4(ou[4], ou[5], ou[6], ou[7]);
    }
    return;
  }
  if (swiglu) {
    // columns [n0, n0+16) are gate, [n0+16, n0+32) are up; N is a multiple of 32 here.
    if (p.D2 != nullptr) {
      uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.D2) + drow * p.ldd2 + n0);
#pragma unroll
      for (int q = 0; q < 4; ++q)
        dst[q] = make_uint4(pack_bf16x2(v[8 * q + 0], v[8 * q + 1]), pack_bf16x2(v[8 * q + 2], v[8 * q + 3]),
                            pack_bf16x2(v[8 * q + 4], v[8 * q + 5]), pack_bf16x2(v[8 * q + 6], v[8 * q + 7]));
    }
    float h[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      // round gate and up to bf16 first so that the result equals the unfused path
      const float g = __bfloat162float(__float2bfloat16(v[j]));
      const float u = __bfloat162float(__float2bfloat16(v[16 + j]));
      h[j] = silu_f(g) * u;
    }
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.D) + drow * p.ldd + (n0 >> 1));
#pragma unroll
    for (int q = 0; q < 2; ++q)
      dst[q] = make_uint4(pack_bf16x2(h[8 * q + 0], h[8 * q + 1]), pack_bf16x2(h[8 * q + 2], h[8 * q + 3]),
                          pack_bf16x2(h[8 * q + 4], h[8 * q + 5]), pack_bf16x2(h[8 * q + 6], h[8 * q + 7]));
    return;
  }
  if (flags & GEMM_ACT_GELU) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = gelu_erf(v[j]);
  }
  if (p.residual != nullptr && !zero_row) {
    const __nv_bfloat16* rs = p.residual + drow * p.ldr + n0;
    if (nvalid == 32 && (p.ldr & 7) == 0 && (reinterpret_cast<uintptr_t>(p.residual) & 15) == 0) {
      const uint4* rs4 = reinterpret_cast<const uint4*>(rs);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint4 x = rs4[q];
        const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(xb[e]);
          v[8 * q + 2 * e] += f.x;
          v[8 * q + 2 * e + 1] += f.y;
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < nvalid) v[j] += __bfloat162float(rs[j]);
    }
  }
  if (out_fp32) {
    float* dst = reinterpret_cast<float*>(p.D) + drow * p.ldd + n0;
    if (nvalid == 32 && (p.ldd & 3) == 0 && (reinterpret_cast<uintptr_t>(p.D) & 15) == 0) {
      float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        float4 o = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        if (accum) {
          const float4 old = d4[q];
          o.x += old.x;
          o.y += old.y;
          o.z += old.z;
          o.w += old.w;
        }
        d4[q] = o;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < nvalid) dst[j] = accum ? dst[j] + v[j] : v[j];
    }
  } else {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.D) + drow * p.ldd + n0;
    if (nvalid == 32 && (p.ldd & 7) == 0 && (reinterpret_cast<uintptr_t>(p.D) & 15) == 0) {
      uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (accum) {
          const uint4 x = d4[q];
          const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(xb[e]);
            v[8 * q + 2 * e] += f.x;
            v[8 * q + 2 * e + 1] += f.y;
          }
        }
        d4[q] = make_uint4(pack_bf16x2(v[8 * q + 0], v[8 * q + 1]), pack_bf16x2(v[8 * q + 2], v[8 * q + 3]),
                           pack_bf16x2(v[8 * q + 4], v[8 * q + 5]), pack_bf16x2(v[8 * q + 6], v[8 * q + 7]));
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < nvalid) dst[j] = __float2bfloat16(accum ? __bfloat162float(dst[j]) + v[j] : v[j]);
    }
  }
}

// Epilogue of one warp for one output tile: the warp's 32 accumulator rows (TMEM lanes of its
// quarter, BN fp32 columns starting at taddr0) go through bias / activation / residual / row map /
// accumulate and are stored. `row_in_prob` is this thread's row within the problem; the warp
// handles the 32-column chunks [chunk0, chunk1) (two warps share a lane quarter).
template <int BN>
__device__ __forceinline__ void epilogue_rows(const Problem& p, int M, int m0, int row_in_prob, int n_base,
                                              uint32_t taddr0, int chunk0, int chunk1) {
  const bool row_ok = row_in_prob < M;
  long drow = static_cast<long>(m0) + row_in_prob;
  // Rows between M and the end of the 128-row tile are zero-filled on request, so that a
  // 128-aligned token segment can later be reduced over without reading garbage.
  // (A 256-row pair tile can reach past that boundary into the next segment: those rows are left alone.)
  const bool zero_row = !row_ok && (p.flags & GEMM_ZERO_PAD_ROWS) != 0 && p.row_map == nullptr &&
                        row_in_prob < ((M + BM - 1) & ~(BM - 1));
  bool store_ok = row_ok || zero_row;
  if (row_ok && p.row_map != nullptr) {
    const int r = p.row_map[drow];
    store_ok = r >= 0;
    drow = r;
  }
  // debug build: the destination row lies inside D (after the row map, with zero-filled pad rows included)
  if (store_ok && !WX_CHK(drow >= 0 && (p.d_rows == 0 || drow < p.d_rows), 2005, drow, p.d_rows)) store_ok = false;

#pragma unroll 1
  for (int c = chunk0; c < chunk1; ++c) {
    uint32_t r[32];
    tmem_ld_32x32(taddr0 + c * 32, r);
    tmem_ld_wait();
    const int n0 = n_base + c * 32;
    if (!store_ok || n0 >= p.N) continue;
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = zero_row ? 0.f : __uint_as_float(r[j]);
    epilogue_chunk(p, v, drow, n0, zero_row);
  }
}

// Copies the weight tiles from the ranks that own them into this GPU's staging buffer; run by one
// thread of a puller CTA. Global -> shared by bulk copy (mbarrier completion), shared -> global by
// bulk store (bulk-group completion), kAgDepth loads in flight. All pullers share every tile
// (chunk i of a tile goes to puller i mod n_pullers), so the first tile arrives as early as the
// links allow; each puller adds 1 to the tile's flag once its part is in memory. The loop is
// scalar code on one thread, so it works in 32-bit chunk units and avoids 64-bit divisions.
struct AgCursor {
  int j, i, nt, n;  // logical tile, chunk in tile, physical tile, chunks in that tile
};

__device__ __forceinline__ void ag_enter(const AgDev& ag, AgCursor& c) {
  int nt = c.j + ag.rot;
  if (nt >= ag.ntiles) nt -= ag.ntiles;
  c.nt = nt;
  c.n = (nt == ag.ntiles - 1) ? ag.last_chunks : ag.cpt;
}

__device__ bool ag_pull(const AgDev& ag, int q, uint8_t* ring, uint64_t* bars, volatile int* abort_flag, int& seq) {
  const int np = ag.n_pullers;
  const uint32_t cb = static_cast<uint32_t>(ag.chunk_bytes);
  int issued = seq, stored = seq;  // chunk sequence numbers of this puller (all stores up to seq are complete)
  int lbuf = seq % kAgRing, sbuf = lbuf;
  uint32_t sphase = (seq / kAgRing) & 1u;
  // tiles whose last store has been issued but not yet confirmed complete
  int pend_tile[kAgPend], pend_seq[kAgPend];
  int pend_head = 0, pend_n = 0;
  AgCursor L{0, q, 0, 0}, S{0, q, 0, 0};
  ag_enter(ag, L);
  ag_enter(ag, S);
  bool ok = true;
  while (true) {
    // load cursor: skip tiles in which this puller has no (more) chunks
    while (L.j < ag.ntiles && L.i >= L.n) {
      L.i = q;
      if (++L.j < ag.ntiles) ag_enter(ag, L);
    }
    const bool loads_done = L.j >= ag.ntiles;
    if (stored < issued && (issued - stored >= kAgDepth || loads_done)) {
      // ---- store side: tiles without a chunk of this puller still get their arrival
      while (S.i >= S.n) {
        red_release_gpu_add(&ag.flags[S.nt], 1);
        S.i = q;
        ++S.j;
        ag_enter(ag, S);
      }
      if (!mbar_wait(&bars[sbuf], sphase, abort_flag)) {
        ok = false;
        break;
      }
      const size_t off = (static_cast<size_t>(S.nt) * ag.cpt + S.i) * cb;
      if (!WX_CHK(S.nt >= 0 && S.nt < ag.ntiles && off + cb <= static_cast<size_t>(ag.total_bytes), 2001, S.nt, off)) {
        ok = false;
        break;
      }
      bulk_store(ag.staging + off, ring + sbuf * kAgChunkMax, cb);
      tma_store_commit();
      ++stored;
      if (++sbuf == kAgRing) {
        sbuf = 0;
        sphase ^= 1u;
      }
      S.i += np;
      // tiles whose stores are certainly complete: kAgLag or more groups were committed after theirs
      if (pend_n > 0 && stored - pend_seq[pend_head] >= kAgLag) {
        bulk_store_wait<kAgLag>();
        fence_proxy_async_global();
        while (pend_n > 0 && stored - pend_seq[pend_head] >= kAgLag) {
          red_release_gpu_add(&ag.flags[pend_tile[pend_head]], 1);
          pend_head = (pend_head + 1) & (kAgPend - 1);
          --pend_n;
        }
      }
      if (S.i >= S.n) {  // last chunk of this puller in the tile: publish once its stores have landed
        if (pend_n == kAgPend) {  // queue full: drain
          bulk_store_wait_all();
          fence_proxy_async_global();
          while (pend_n > 0) {
            red_release_gpu_add(&ag.flags[pend_tile[pend_head]], 1);
            pend_head = (pend_head + 1) & (kAgPend - 1);
            --pend_n;
          }
        }
        const int slot = (pend_head + pend_n) & (kAgPend - 1);
        pend_tile[slot] = S.nt;
        pend_seq[slot] = stored;
        ++pend_n;
        S.i = q;
        if (++S.j < ag.ntiles) ag_enter(ag, S);
        else S.n = 0x7fffffff;  // nothing left: the store side is only entered again with a loaded chunk
      }
      continue;
    }
    if (loads_done) break;
    // ---- load side
    if (issued - seq >= kAgRing) bulk_store_wait_read<2>();  // the store that last read this buffer is 2+ groups back
    const uint32_t g = static_cast<uint32_t>(L.nt) * ag.cpt + L.i;  // chunk index in the whole weight
    const uint32_t r = g / static_cast<uint32_t>(ag.cps);
    if (!WX_CHK(r < 8u && ag.peer[r] != nullptr && static_cast<long>(g - r * ag.cps + 1) * cb <= ag.shard_bytes, 2002, g, r)) {
      ok = false;
      break;
    }
    const uint8_t* src = ag.peer[r] + static_cast<size_t>(g - r * ag.cps) * cb;
    mbar_arrive_expect_tx(&bars[lbuf], cb);
    bulk_load(ring + lbuf * kAgChunkMax, src, cb, &bars[lbuf]);
    ++issued;
    if (++lbuf == kAgRing) lbuf = 0;
    L.i += np;
  }
  bulk_store_wait_all();
  fence_proxy_async_global();
  if (ok) {
    while (pend_n > 0) {
      red_release_gpu_add(&ag.flags[pend_tile[pend_head]], 1);
      pend_head = (pend_head + 1) & (kAgPend - 1);
      --pend_n;
    }
    // trailing tiles without a chunk of this puller
    while (S.j < ag.ntiles) {
      if (S.n != 0x7fffffff) red_release_gpu_add(&ag.flags[S.nt], 1);
      S.i = q;
      if (++S.j < ag.ntiles) ag_enter(ag, S);
    }
  }
  seq = issued;
  return ok;
}

// Bounded wait of a GEMM producer for a gathered tile.
__device__ __forceinline__ bool ag_wait(const int* flag, int target, volatile int* abort_flag) {
  if (!WX_CHK(flag != nullptr && target > 0, 2003, target, 0)) {
    *abort_flag = 1;
    return false;
  }
  if (ld_acquire_gpu(flag) < target) {
    const long long t0 = clock64();
    while (ld_acquire_gpu(flag) < target) {
      if (*abort_flag) return false;
      if (clock64() - t0 > WX_WAIT_LIMIT_CYCLES) {
        *abort_flag = 1;
        return false;
      }
      __nanosleep(64);
    }
  }
  fence_proxy_async_global();
  return true;
}

template <int BN, bool A_MN, bool B_MN, bool AG>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ GemmArgs args, int* __restrict__ status) {
  using C = Cfg<BN>;
  static_assert(!AG || BN == 256, "copy CTAs: 256-wide tiles only");
  static_assert(!AG || C::STAGES * C::STAGE_BYTES >= kAgRing * kAgChunkMax, "ring must fit in the stage area");
  const int n_pull = AG ? args.ag[0].n_pullers : 0;
  const bool puller = AG && static_cast<int>(blockIdx.x) < n_pull;
  const int cta = static_cast<int>(blockIdx.x) - n_pull;
  const int ncta = static_cast<int>(gridDim.x) - n_pull;
  const bool gathered = AG && args.ag_wait != 0;  // B operands arrive while the kernel runs
  const int rot0 = (gathered && !B_MN) ? args.ag[0].rot : 0;
  const int rot1 = (gathered && !B_MN) ? args.ag[1].rot : 0;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
  uint64_t* empty_bar = full_bar + C::STAGES;
  uint64_t* tfull_bar = empty_bar + C::STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    if (puller) {
      // the 2 * STAGES + 4 barriers are contiguous; a puller uses the first kAgRing of them
      static_assert(!AG || 2 * C::STAGES + 4 >= kAgRing, "not enough barriers for the ring");
      for (int s = 0; s < kAgRing; ++s) mbar_init(&full_bar[s], 1);
    } else {
      for (int s = 0; s < C::STAGES; ++s) {
        mbar_init(&full_bar[s], 1);
        mbar_init(&empty_bar[s], 1);
      }
      for (int a = 0; a < 2; ++a) {
        mbar_init(&tfull_bar[a], 1);
        mbar_init(&tempty_bar[a], kEpiWarps);
      }
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == kEpiWarp0) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  Dims d;
  load_dims<BN>(args, d);
  const int total_tiles = d.tiles[0] + d.tiles[1];

  if (puller) {
    if (threadIdx.x == 0) {
      int seq = 0;  // chunk sequence number carries over: the ring's barrier phases continue
      const int n = gathered ? args.nprob : args.n_ag;
      for (int i = 0; i < n; ++i)
        if (!ag_pull(args.ag[i], static_cast<int>(blockIdx.x), smem, full_bar, abort_flag, seq)) break;
    }
  } else if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int i = 0; i < args.nprob; ++i) {
        tma_prefetch_desc(&args.p[i].tmA);
        tma_prefetch_desc(&args.p[i].tmB);
      }
      int s = 0;
      uint32_t phase = 0;
      bool ok = true;
      int ag_ready[2] = {0, 0};  // MN-major B: 256-row blocks of the weight known to be in place
      for (int t = cta; t < total_tiles && ok; t += ncta) {
        const TileInfo ti = decode_tile(d, t, gathered, rot0, rot1);
        const Problem& p = args.p[ti.prob];
        const int m_base = d.m0[ti.prob] + ti.mt * BM;
        const int n_base = ti.nt * BN;
        const int k_base = d.k0[ti.prob];
        const int nkb = (d.K[ti.prob] + BK - 1) / BK;
        if (!WX_CHK(ti.mt >= 0 && ti.mt < d.tiles_m[ti.prob] && ti.nt >= 0 && ti.nt < d.tiles_n[ti.prob] && (k_base & 7) == 0,
                    2004, ti.mt, ti.nt)) {
          *abort_flag = 1;
          break;
        }
        for (int kb = 0; kb < nkb; ++kb) {
          if (gathered) {
            if (!B_MN) {
              if (kb == 0 && !ag_wait(&args.ag[ti.prob].flags[ti.nt], args.ag[ti.prob].target, abort_flag)) {
                ok = false;
                break;
              }
            } else {
              const int blk = (k_base + kb * BK + BK - 1) >> 8;
              if (blk >= ag_ready[ti.prob]) {
                if (!ag_wait(&args.ag[ti.prob].flags[blk], args.ag[ti.prob].target, abort_flag)) {
                  ok = false;
                  break;
                }
                ag_ready[ti.prob] = blk + 1;  // pullers finish tiles in order
              }
            }
          }
          if (!mbar_wait(&empty_bar[s], phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          uint8_t* sA = smem + s * C::STAGE_BYTES;
          uint8_t* sB = sA + C::A_BYTES;
          mbar_arrive_expect_tx(&full_bar[s], C::STAGE_BYTES);
          const int kc = k_base + kb * BK;
          if (!A_MN) {
            tma_load_2d(sA, &p.tmA, &full_bar[s], kc, m_base);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(sA + j * 8192, &p.tmA, &full_bar[s], m_base + 64 * j, kc);
          }
          if (!B_MN) {
            tma_load_2d(sB, &p.tmB, &full_bar[s], kc, n_base);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(sB + j * 8192, &p.tmB, &full_bar[s], n_base + 64 * j, kc);
          }
          if (++s == C::STAGES) {
            s = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      int s = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = cta; t < total_tiles && ok; t += ncta, ++it) {
        const TileInfo ti = decode_tile(d, t, gathered, rot0, rot1);
        const int nkb = (d.K[ti.prob] + BK - 1) / BK;
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, abort_flag)) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&full_bar[s], phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * C::STAGE_BYTES);
          const uint32_t b_addr = a_addr + C::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = A_MN ? make_smem_desc_sw128(a_addr + k * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(a_addr + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc_sw128(b_addr + k * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(b_addr + k * 32, 16, 1024);
            tc_mma_bf16(tmem_d, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit(&empty_bar[s]);
          if (++s == C::STAGES) {
            s = 0;
            phase ^= 1u;
          }
        }
        if (ok) tc_commit(&tfull_bar[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quarter = warp & 3;  // TMEM lane quarter this warp may read
    const int half = (warp - kEpiWarp0) >> 2;  // which half of the tile's columns
    constexpr int kChunks = BN / 32;
    const int chunk0 = (kChunks >= 2) ? half * (kChunks / 2) : 0;
    const int chunk1 = (kChunks >= 2) ? chunk0 + kChunks / 2 : (half == 0 ? 1 : 0);
    int it = 0;
    for (int t = cta; t < total_tiles; t += ncta, ++it) {
      const TileInfo ti = decode_tile(d, t, gathered, rot0, rot1);
      const Problem& p = args.p[ti.prob];
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag)) break;
      tc_fence_after();

      epilogue_rows<BN>(p, d.M[ti.prob], d.m0[ti.prob], ti.mt * BM + quarter * 32 + lane, ti.nt * BN,
                        tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16), chunk0, chunk1);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicExch(status, 1);
  if (warp == kEpiWarp0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// --------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
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

// cuTensorMapEncodeTiled is a driver call and needs a context bound to the calling thread. A
// thread whose first CUDA work is one of these launches (an autograd worker on device 0, for
// which torch skips cudaSetDevice) has none yet; cudaFree(nullptr) makes the runtime bind the
// primary context.
void bind_context_once() {
  thread_local bool bound = false;
  if (!bound) {
    cudaFree(nullptr);
    bound = true;
  }
}

// 2-D bf16 tensor map with 128-byte swizzle; `inner` is the contiguous extent.
bool make_tmap(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint64_t pitch_elems,
               uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return false;
  bind_context_once();
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {pitch_elems * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

int num_sms() { return sm_count(); }

template <int BN, bool A_MN, bool B_MN, bool AG = false>
int launch_t(const GemmArgs& args, int grid, cudaStream_t stream, int* status) {
  using C = Cfg<BN>;
  auto kern = gemm_kernel<BN, A_MN, B_MN, AG>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set = true;
  }
  kern<<<grid, kThreads, C::SMEM_BYTES, stream>>>(args, status);
  return static_cast<int>(cudaGetLastError());
}

template <int BN>
int launch_bn(const GemmArgs& args, bool a_mn, bool b_mn, int grid, cudaStream_t stream, int* status) {
  if (!a_mn && !b_mn) return launch_t<BN, false, false>(args, grid, stream, status);
  if (!a_mn && b_mn) return launch_t<BN, false, true>(args, grid, stream, status);
  if (a_mn && !b_mn) return launch_t<BN, true, false>(args, grid, stream, status);
  return launch_t<BN, true, true>(args, grid, stream, status);
}

int fill_args(GemmArgs& args, const GemmCall* calls, int ncalls, int bn, int a_rows = BM) {
  args.nprob = ncalls;
  {
    static const int env_group = [] {
      const char* e = getenv("WX_RASTER_GROUP");
      return e ? atoi(e) : 0;
    }();
    args.raster_group = env_group;
  }
  args.ag[0] = AgDev{};
  args.ag[1] = AgDev{};
  args.ag_wait = 1;
  args.n_ag = 0;
  for (int i = 0; i < ncalls; ++i) {
    const GemmCall& c = calls[i];
    Problem& p = args.p[i];
    bool ok;
    if (!c.a_mn)
      ok = make_tmap(&p.tmA, c.A, c.a_extent_k, c.a_extent_mn, c.lda, BK, a_rows);
    else
      ok = make_tmap(&p.tmA, c.A, c.a_extent_mn, c.a_extent_k, c.lda, 64, BK);
    if (!ok) return -4;
    if (!c.b_mn)
      ok = make_tmap(&p.tmB, c.B, c.b_extent_k, c.b_extent_mn, c.ldb, BK, bn);
    else
      ok = make_tmap(&p.tmB, c.B, c.b_extent_mn, c.b_extent_k, c.ldb, 64, BK);
    if (!ok) return -5;
    p.D = c.D;
    p.D2 = c.D2;
    p.bias = reinterpret_cast<const __nv_bfloat16*>(c.bias);
    p.residual = reinterpret_cast<const __nv_bfloat16*>(c.residual);
    p.row_map = c.row_map;
    p.dyn = c.dyn;
    p.ldd = c.ldd;
    p.d_rows = c.d_rows;
    p.ldd2 = c.ldd2;
    p.ldr = c.ldr;
    p.M = c.M;
    p.N = c.N;
    p.K = c.K;
    p.m0 = c.m0;
    p.k0 = c.k0;
    p.flags = c.flags;
  }
  return 0;
}

// Device view of one gather: chunking of the weight's byte run, flag target of this epoch, starting tile.
int fill_ag_dev(AgDev& a, const AgInfo& ag, long w_rows, long w_cols, int np, bool b_mn) {
  for (int r = 0; r < ag.world; ++r) a.peer[r] = static_cast<const uint8_t*>(ag.peer[r]);
  a.staging = static_cast<uint8_t*>(ag.staging);
  a.flags = ag.flags;
  a.shard_bytes = static_cast<long>(ag.rows_per_rank) * w_cols * 2;
  a.tile_bytes = 256 * w_cols * 2;
  a.total_bytes = w_rows * w_cols * 2;
  a.ntiles = static_cast<int>((w_rows + 255) / 256);
  // chunk: the largest multiple of 16 bytes, at most 16 KB, dividing both the shard and the tile
  int chunk = 0;
  for (int c = kAgChunkMax; c >= 16; c -= 16)
    if (a.shard_bytes % c == 0 && a.tile_bytes % c == 0) {
      chunk = c;
      break;
    }
  if (chunk == 0) return -9;
  a.chunk_bytes = chunk;
  a.cpt = static_cast<int>(a.tile_bytes / chunk);
  a.last_chunks = static_cast<int>((a.total_bytes - static_cast<long>(a.ntiles - 1) * a.tile_bytes) / chunk);
  a.cps = static_cast<int>(a.shard_bytes / chunk);
  a.n_pullers = np;
  a.target = np * ag.epoch;
  a.rot = b_mn ? 0 : static_cast<int>((static_cast<long>(ag.rank) * ag.rows_per_rank) / 256) % a.ntiles;
  return 0;
}

}  // namespace

WX_CHK_DEFINE_READER(gemm_check_read)
int gemm_checked_build() { return WX_CHECKED_BUILD; }

}  // namespace wx

#include "gemm2.cuh"
#include "gemm_skinny.cuh"

namespace wx {

namespace {
// TFLOP/s of the 128 x {256, 128, 64} single-CTA tiles and of the 256 x 256 CTA-pair tile on a large problem.
double g_tile_rates[4] = {1260.0, 970.0, 525.0, 1360.0};
}  // namespace

void gemm_set_tile_rates(const double* rates4) {
  for (int i = 0; i < 4; ++i)
    if (rates4[i] > 0.0) g_tile_rates[i] = rates4[i];
}
void gemm_get_tile_rates(double* rates4) {
  for (int i = 0; i < 4; ++i) rates4[i] = g_tile_rates[i];
}

int gemm_launch(const GemmCall* calls, int ncalls, cudaStream_t stream, int* status, int force_bn) {
  if (ncalls < 1 || ncalls > 2) return -1;
  const bool a_mn = calls[0].a_mn, b_mn = calls[0].b_mn;
  for (int i = 1; i < ncalls; ++i)
    if (calls[i].a_mn != a_mn || calls[i].b_mn != b_mn) return -2;

  // Few rows (decode, denoise steps): clusters of CTAs that split K (gemm_skinny.cuh). force_bn = 16 selects that
  // kernel where it is legal, 17 the same with one CTA per column tile (no split); other forced widths bypass it.
  // force_bn = 18 is "automatic, inference": it also lets problems of up to 1024 rows whose 128 x 256 tiles fill less
  // than half of the SMs and whose K is 4096 or more run on K-splitting clusters (prefix passes: few tiles, long K, one
  // serial chain per tile).
  // Training launches (0) take neither that second path nor a K split of the few-row kernel, so a different summation
  // order cannot enter a comparison of training runs.
  const bool infer = force_bn == 18;
  if (infer) force_bn = 0;
  if (!a_mn && !b_mn && (force_bn == 0 || force_bn == 16 || force_bn == 17)) {
    int max_m = 0, min_nkb = 1 << 30;
    long st = 0, mid = 0;
    bool plain = true;
    for (int i = 0; i < ncalls; ++i) {
      max_m = calls[i].M > max_m ? calls[i].M : max_m;
      st += (calls[i].N + kSkinnyBN - 1) / kSkinnyBN;
      mid += static_cast<long>((calls[i].N + kMidBN - 1) / kMidBN) * ((calls[i].M + BM - 1) / BM);
      const int nkb = (calls[i].K + BK - 1) / BK;
      min_nkb = nkb < min_nkb ? nkb : min_nkb;
      if ((calls[i].flags & (GEMM_ACT_SWIGLU | GEMM_SWIGLU_BWD)) && (calls[i].N % 32 != 0)) plain = false;
      if (calls[i].flags & GEMM_ZERO_PAD_ROWS) plain = false;  // rows past M are never visited by that kernel
    }
    if (plain && max_m >= 1 && max_m <= BM && st >= 1 && st <= 1024) {
      GemmArgs sargs;
      const int a_rows = skinny_rows(max_m);
      const int src = fill_args(sargs, calls, ncalls, kSkinnyBN, a_rows);
      if (src != 0) return src;
      // K is split over a cluster for inference launches only: a training launch must give the bits of the general
      // kernel (the fused-gather GEMM of a row-sharded weight is that kernel, and the plans are compared bit for bit)
      const int splits = (infer || force_bn == 16) ? skinny_splits(st, min_nkb, num_sms()) : 1;
      return launch_skinny(sargs, a_rows, kSkinnyBN, static_cast<int>(st), splits, stream, status);
    }
    if (force_bn == 16 || force_bn == 17) return -11;
    // (measured in CUDA graphs at 314 rows: 35 against 54 us for K = 11008, but 24 against 15 us for K = 2048, where the
    // hand-over and reduction of 128 x 256 partial tiles costs more than the shorter chain saves: long K only)
    static const int mid_min_nkb = [] {
      const char* e = getenv("WX_MID_MIN_NKB");
      return e ? atoi(e) : 64;
    }();
    if (infer && plain && max_m > BM && max_m <= 1024 && mid >= 1 && min_nkb >= mid_min_nkb) {
      const int splits = skinny_splits(mid, min_nkb, num_sms());
      if (splits >= 2) {
        GemmArgs sargs;
        const int src = fill_args(sargs, calls, ncalls, kMidBN, BM);
        if (src != 0) return src;
        return launch_skinny(sargs, BM, kMidBN, static_cast<int>(mid), splits, stream, status);
      }
    }
  }

  const int sms = num_sms();
  auto count_tiles = [&](int bn) {
    long t = 0;
    for (int i = 0; i < ncalls; ++i)
      t += static_cast<long>((calls[i].M + BM - 1) / BM) * ((calls[i].N + bn - 1) / bn);
    return t;
  };
  // Tile width: minimise (number of waves) x (time of one tile). The per-width rates (TFLOP/s with every SM busy) come
  // from g_tile_rates: measured once per process on the device in use (gemm_set_tile_rates, called by
  // ops.gemm.calibrate_tile_rates), with the figures of one B200 as the start-up values.
  int bn = 64;
  bool use_pair = force_bn == 512;
  if (force_bn == 64 || force_bn == 128 || force_bn == 256 || (force_bn == 32 && !a_mn && !b_mn)) {
    bn = force_bn;
  } else if (!use_pair) {
    int max_n = 0;
    for (int i = 0; i < ncalls; ++i) max_n = calls[i].N > max_n ? calls[i].N : max_n;
    const int widths[3] = {256, 128, 64};
    const double eff[3] = {g_tile_rates[0], g_tile_rates[1], g_tile_rates[2]};
    const double bias[3] = {1.0, 1.12, 1.25};  // wave counting is crude: prefer the wider tile on near ties
    double best = 1e300;
    for (int w = 0; w < 3; ++w) {
      if (widths[w] > 64 && max_n <= widths[w] / 2) continue;  // mostly padding
      const long t = count_tiles(widths[w]);
      const long waves = (t + sms - 1) / sms;
      const double cost = static_cast<double>(waves) * widths[w] / eff[w] * bias[w];
      if (cost < best) {
        best = cost;
        bn = widths[w];
      }
    }
    // CTA pairs (256 x 256 tiles, one per two SMs): same work per SM and tile as the 128 x 256
    // kernel at about 1.08x its rate; chosen when its wave count does not eat that up.
    if (max_n > 128) {
      long pt = 0;
      for (int i = 0; i < ncalls; ++i)
        pt += static_cast<long>((calls[i].M + 255) / 256) * ((calls[i].N + 255) / 256);
      const long pairs = sms / 2;
      const long pwaves = (pt + pairs - 1) / pairs;
      const double pcost = static_cast<double>(pwaves) * 256 / g_tile_rates[3];
      if (pcost < best) use_pair = true;
    }
  }
  // (32-wide tiles exist for K-major operands and can be forced; measured on decode-sized problems they
  // are not faster than 64-wide ones -- the 128-row A tile dominates each step -- so they are never chosen.)
  for (int i = 0; i < ncalls; ++i)
    if ((calls[i].flags & (GEMM_ACT_SWIGLU | GEMM_SWIGLU_BWD)) && (calls[i].N % 32 != 0)) return -3;

  if (use_pair) {  // CTA pairs: 256 x 256 tiles
    GemmArgs pargs;
    const int prc = fill_args(pargs, calls, ncalls, 128);
    if (prc != 0) return prc;
    long ptiles = 0;
    for (int i = 0; i < ncalls; ++i)
      ptiles += static_cast<long>((calls[i].M + 255) / 256) * ((calls[i].N + 255) / 256);
    if (ptiles <= 0) return 0;
    const int prc2 = launch_pair(pargs, a_mn, b_mn, ptiles, stream, status);
    if (prc2 != -10 || force_bn == 512) return prc2;  // -10: clusters cannot be scheduled here -> single-CTA kernel
  }

  GemmArgs args;
  const int rc = fill_args(args, calls, ncalls, bn);
  if (rc != 0) return rc;
  long tiles = count_tiles(bn);
  if (tiles <= 0) return 0;
  int grid = tiles < sms ? static_cast<int>(tiles) : sms;
  if (bn == 256) return launch_bn<256>(args, a_mn, b_mn, grid, stream, status);
  if (bn == 128) return launch_bn<128>(args, a_mn, b_mn, grid, stream, status);
  if (bn == 32) return launch_t<32, false, false>(args, grid, stream, status);
  return launch_bn<64>(args, a_mn, b_mn, grid, stream, status);
}

int gemm_ag_launch(const GemmCall* calls, const AgInfo* ags, int ncalls, cudaStream_t stream, int* status) {
  if (ncalls < 1 || ncalls > 2) return -1;
  const bool b_mn = calls[0].b_mn;
  for (int i = 0; i < ncalls; ++i)
    if (calls[i].a_mn || calls[i].b_mn != b_mn) return -2;
  for (int i = 0; i < ncalls; ++i)
    if ((calls[i].flags & (GEMM_ACT_SWIGLU | GEMM_SWIGLU_BWD)) && (calls[i].N % 32 != 0)) return -3;
  GemmArgs args;
  const int rc = fill_args(args, calls, ncalls, 256);
  if (rc != 0) return rc;
  const int sms = num_sms();
  int np = ags[0].n_pullers > 0 ? ags[0].n_pullers : 8;
  np = (np + 1) & ~1;  // even: on CTA pairs whole clusters copy, and both kernels must count the same arrivals per tile
  if (np > sms / 2) np = (sms / 2) & ~1;
  long tiles = 0;
  for (int i = 0; i < ncalls; ++i) {
    const GemmCall& call = calls[i];
    const AgInfo& ag = ags[i];
    if (ag.world < 1 || ag.world > 8 || ag.rows_per_rank < 1 || ag.epoch < 1) return -6;
    if (call.B != ag.staging) return -7;
    // rows of the weight in memory, and its row length
    const long w_rows = static_cast<long>(ag.world) * ag.rows_per_rank;
    const long w_cols = call.ldb;
    if (!b_mn ? (w_rows != call.N || call.b_extent_mn != w_rows) : (call.b_extent_k != w_rows)) return -8;
    if ((w_cols * 2) % 16 != 0) return -9;
    for (int r = 0; r < ag.world; ++r)
      if (ag.peer[r] == nullptr || (reinterpret_cast<uintptr_t>(ag.peer[r]) & 15) != 0) return -9;
    if ((reinterpret_cast<uintptr_t>(ag.staging) & 15) != 0) return -9;
    const int frc = fill_ag_dev(args.ag[i], ag, w_rows, w_cols, np, b_mn);
    if (frc != 0) return frc;
    tiles += static_cast<long>((call.M + BM - 1) / BM) * ((call.N + 255) / 256);
  }
  if (tiles <= 0) return 0;
  // CTA pairs (256 x 256 tiles) when the problem has enough of them to fill the pairs that remain beside the copy
  // CTAs; the tensor maps then use 128-row B boxes (each CTA of a pair loads its half of the 256 weight rows)
  {
    // opt-in (WX_AG_PAIR=1) until it has been timed against the single-CTA gathered kernel on more than one GPU
    static const bool pair_ok = [] {
      const char* e = getenv("WX_AG_PAIR");
      return e != nullptr && atoi(e) != 0;
    }();
    long ptiles = 0;
    int max_n = 0;
    for (int i = 0; i < ncalls; ++i) {
      ptiles += static_cast<long>((calls[i].M + 255) / 256) * ((calls[i].N + 255) / 256);
      max_n = calls[i].N > max_n ? calls[i].N : max_n;
    }
    const int np2 = np;  // even (see above): whole clusters copy
    if (pair_ok && max_n > 128 && ptiles >= (sms - np2) / 2) {
      GemmArgs pargs;
      if (fill_args(pargs, calls, ncalls, 128) == 0) {
        pargs.ag[0] = args.ag[0];
        pargs.ag[1] = args.ag[1];
        for (int i = 0; i < ncalls; ++i) {
          pargs.ag[i].n_pullers = np2;
          pargs.ag[i].target = np2 * ags[i].epoch;
        }
        const int prc = b_mn ? launch_pair_ag_t<false, true>(pargs, ptiles, np2, stream, status)
                             : launch_pair_ag_t<false, false>(pargs, ptiles, np2, stream, status);
        if (prc != -10) return prc;
      }
    }
  }
  const int workers = tiles < sms - np ? static_cast<int>(tiles) : sms - np;
  const int grid = workers + np;
  if (!b_mn) return launch_t<256, false, false, true>(args, grid, stream, status);
  return launch_t<256, false, true, true>(args, grid, stream, status);
}

// One or two GEMM problems whose operands are all in place, plus up to two weight gathers that the launch's copy CTAs
// run for LATER launches (ags[i].staging is filled from ags[i].peer; `cols[i]` is weight i's row length in elements).
// Nothing in this launch waits for the gathers: a kernel launched afterwards on the same stream may read the staging
// buffers as plain operands. Used in backward: the weight-gradient GEMM of one projection (which needs no weight)
// carries the gather of the weight that the next dgrad GEMM multiplies by, so that gather costs no time of its own.
int gemm_launch_prefetch(const GemmCall* calls, int ncalls, const AgInfo* ags, const long* cols, int n_ags, cudaStream_t stream,
                         int* status) {
  if (ncalls < 1 || ncalls > 2 || n_ags < 1 || n_ags > 2) return -1;
  const bool a_mn = calls[0].a_mn, b_mn = calls[0].b_mn;
  for (int i = 1; i < ncalls; ++i)
    if (calls[i].a_mn != a_mn || calls[i].b_mn != b_mn) return -2;
  for (int i = 0; i < ncalls; ++i)
    if ((calls[i].flags & (GEMM_ACT_SWIGLU | GEMM_SWIGLU_BWD)) && (calls[i].N % 32 != 0)) return -3;
  const int sms = num_sms();
  int np = ags[0].n_pullers > 0 ? ags[0].n_pullers : 8;
  np = (np + 1) & ~1;
  if (np > sms / 2) np = (sms / 2) & ~1;
  AgDev devs[2] = {AgDev{}, AgDev{}};
  for (int i = 0; i < n_ags; ++i) {
    const AgInfo& ag = ags[i];
    if (ag.world < 1 || ag.world > 8 || ag.rows_per_rank < 1 || ag.epoch < 1 || cols[i] < 8 || (cols[i] * 2) % 16 != 0) return -6;
    for (int r = 0; r < ag.world; ++r)
      if (ag.peer[r] == nullptr || (reinterpret_cast<uintptr_t>(ag.peer[r]) & 15) != 0) return -9;
    if (ag.staging == nullptr || (reinterpret_cast<uintptr_t>(ag.staging) & 15) != 0) return -9;
    const int frc = fill_ag_dev(devs[i], ag, static_cast<long>(ag.world) * ag.rows_per_rank, cols[i], np, true);
    if (frc != 0) return frc;
  }
  long ptiles = 0, tiles = 0;
  int max_n = 0;
  for (int i = 0; i < ncalls; ++i) {
    ptiles += static_cast<long>((calls[i].M + 255) / 256) * ((calls[i].N + 255) / 256);
    tiles += static_cast<long>((calls[i].M + BM - 1) / BM) * ((calls[i].N + 255) / 256);
    max_n = calls[i].N > max_n ? calls[i].N : max_n;
  }
  if (tiles <= 0) return -1;
  auto finish = [&](GemmArgs& a) {
    a.ag[0] = devs[0];
    a.ag[1] = devs[1];
    a.ag_wait = 0;
    a.n_ag = n_ags;
  };
  if (max_n > 128 && ptiles >= (sms - np) / 4) {  // CTA pairs unless the problem is tiny
    GemmArgs pargs;
    if (fill_args(pargs, calls, ncalls, 128) == 0) {
      finish(pargs);
      int prc = -10;
      if (!a_mn && !b_mn) prc = launch_pair_ag_t<false, false>(pargs, ptiles, np, stream, status);
      else if (!a_mn && b_mn) prc = launch_pair_ag_t<false, true>(pargs, ptiles, np, stream, status);
      else if (a_mn && b_mn) prc = launch_pair_ag_t<true, true>(pargs, ptiles, np, stream, status);
      if (prc != -10) return prc;
    }
  }
  GemmArgs args;
  const int rc = fill_args(args, calls, ncalls, 256);
  if (rc != 0) return rc;
  finish(args);
  const int workers = tiles < sms - np ? static_cast<int>(tiles) : sms - np;
  const int grid = workers + np;
  if (!a_mn && !b_mn) return launch_t<256, false, false, true>(args, grid, stream, status);
  if (!a_mn && b_mn) return launch_t<256, false, true, true>(args, grid, stream, status);
  if (a_mn && b_mn) return launch_t<256, true, true, true>(args, grid, stream, status);
  return -2;
}

}  // namespace wx
