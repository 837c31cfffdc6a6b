// CTA-pair variant of the GEMM core: one 256 x 256 output tile per pair of SMs
// (`tcgen05.mma.cta_group::2`). Included by gemm.cu after its shared declarations. Serves the same calls as the
// single-CTA kernel (reference: csrc/dual_asym_grouped_gemm.cu:49-136 and the cuBLAS GEMMs behind every nn.Linear).
//
// Why: a 128 x 256 x 64 step of the single-CTA kernel moves 48 KB through one SM's shared memory
// twice (TMA write + operand read), which takes longer than the MMAs themselves; with a pair each
// SM stages its own 128 rows of A and only its 128-row half of B (32 KB per step), and the
// hardware shares the B halves between the two tensor cores.
//
// Layout of the work inside a pair (cluster of 2 CTAs, rank 0 = leader):
//   * both CTAs: warp 0 lane 0 issues the TMA loads of this CTA's A rows and B half into its own
//     shared memory; the byte counts of BOTH CTAs are reported to the leader's `full` barrier
//     (`.cta_group::2` form of the load, no multicast);
//   * leader: warp 1 lane 0 waits on `full`, issues the pair MMAs, and commits to the `empty`
//     barrier of each CTA (two commits; a remote commit uses the peer's shared::cluster address);
//   * both CTAs: warps 2..9 wait on their own `tfull`, run the same epilogue as the single-CTA
//     kernel on their 128 rows, and arrive (16 arrivals per tile) on the leader's `tempty`.
// Every wait is bounded; a CTA that gives up still reaches the final cluster barrier, so its peer
// is never left signalling a CTA that has exited.
#pragma once

namespace wx {
namespace {

constexpr int kPairStages = 6;
constexpr int kPairABytes = BM * BK * 2;           // 128 rows of A, 64 k
constexpr int kPairBBytes = 128 * BK * 2;          // this CTA's 128-row half of B
constexpr int kPairStageBytes = kPairABytes + kPairBBytes;
constexpr int kPairSmemBytes = kPairStages * kPairStageBytes + 1024 + 256;
constexpr int kPairTileM = 2 * BM;
constexpr int kPairTileN = 256;

// AG: the weight operand is gathered from the ranks' shards while the kernel runs (see AgInfo in gemm.h). The first
// `n_pullers` CTAs of the grid (whole clusters, so an even number) copy instead of multiplying: one thread of each
// runs the same bulk-copy ring as in the single-CTA kernel; the GEMM pairs take the 256-row weight tiles in arrival
// order and their producers wait (bounded) on a tile's flag before its first B load.
template <bool A_MN, bool B_MN, bool AG = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ GemmArgs args, int* __restrict__ status) {
  static_assert(!AG || kPairStages * kPairStageBytes >= kAgRing * kAgChunkMax, "ring must fit in the stage area");
  static_assert(!AG || 2 * kPairStages + 4 >= kAgRing, "not enough barriers for the ring");
  const int n_pull = AG ? args.ag[0].n_pullers : 0;
  const bool puller = AG && static_cast<int>(blockIdx.x) < n_pull;
  const bool gathered = AG && args.ag_wait != 0;  // B operands arrive while the kernel runs (else: prefetch only)
  const int rot0 = (gathered && !B_MN) ? args.ag[0].rot : 0;
  const int rot1 = (gathered && !B_MN) ? args.ag[1].rot : 0;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kPairStages * kPairStageBytes);
  uint64_t* empty_bar = full_bar + kPairStages;
  uint64_t* tfull_bar = empty_bar + kPairStages;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    if (puller) {
      for (int s = 0; s < kAgRing; ++s) mbar_init(&full_bar[s], 1);  // the copy ring uses the first barriers
    } else {
      for (int s = 0; s < kPairStages; ++s) {
        mbar_init(&full_bar[s], 1);   // used in the leader only: its producer's arrive + both CTAs' bytes
        mbar_init(&empty_bar[s], 1);  // one commit per use, in each CTA
      }
      for (int a = 0; a < 2; ++a) {
        mbar_init(&tfull_bar[a], 1);   // one commit per tile, in each CTA
        mbar_init(&tempty_bar[a], 2 * kEpiWarps);  // used in the leader only: the epilogue warps of both CTAs
      }
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == kEpiWarp0) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_arrive();  // barriers and tensor memory of both CTAs exist before anything crosses
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  Dims d;
  load_dims<kPairTileN, kPairTileM>(args, d);
  const int total_tiles = d.tiles[0] + d.tiles[1];
  const int pair = (static_cast<int>(blockIdx.x) - n_pull) >> 1;
  const int npair = (static_cast<int>(gridDim.x) - n_pull) >> 1;

  if (puller) {
    if (threadIdx.x == 0) {
      int seq = 0;  // chunk sequence number carries over: the ring's barrier phases continue
      const int n = gathered ? args.nprob : args.n_ag;
      for (int i = 0; i < n; ++i)
        if (!ag_pull(args.ag[i], static_cast<int>(blockIdx.x), smem, full_bar, abort_flag, seq)) break;
    }
  } else if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      for (int i = 0; i < args.nprob; ++i) {
        tma_prefetch_desc(&args.p[i].tmA);
        tma_prefetch_desc(&args.p[i].tmB);
      }
      int s = 0;
      uint32_t phase = 0;
      bool ok = true;
      int ag_ready[2] = {0, 0};  // MN-major B: 256-row blocks of the weight known to be in place
      for (int t = pair; t < total_tiles && ok; t += npair) {
        const TileInfo ti = decode_tile(d, t, gathered, rot0, rot1);
        const Problem& p = args.p[ti.prob];
        const int m_base = d.m0[ti.prob] + ti.mt * kPairTileM + static_cast<int>(rank) * BM;
        const int n_base = ti.nt * kPairTileN + static_cast<int>(rank) * 128;
        const int k_base = d.k0[ti.prob];
        const int nkb = (d.K[ti.prob] + BK - 1) / BK;
        for (int kb = 0; kb < nkb; ++kb) {
          if (gathered) {
            if (!B_MN) {  // the pair's 256 weight rows are one flag tile
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
          uint8_t* sA = smem + s * kPairStageBytes;
          uint8_t* sB = sA + kPairABytes;
          if (leader) mbar_arrive_expect_tx(&full_bar[s], 2 * kPairStageBytes);
          const uint32_t full0 = mapa_u32(smem_u32(&full_bar[s]), 0);
          const int kc = k_base + kb * BK;
          if (!A_MN) {
            tma_load_2d_pair(sA, &p.tmA, full0, kc, m_base);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sA + j * 8192, &p.tmA, full0, m_base + 64 * j, kc);
          }
          if (!B_MN) {
            tma_load_2d_pair(sB, &p.tmB, full0, kc, n_base);
          } else {
#pragma unroll
            for (int j = 0; j < 2; ++j) tma_load_2d_pair(sB + j * 8192, &p.tmB, full0, n_base + 64 * j, kc);
          }
          if (++s == kPairStages) {
            s = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader only)
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = make_idesc_bf16(kPairTileM, kPairTileN, A_MN, B_MN);
      int s = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = pair; t < total_tiles && ok; t += npair, ++it) {
        const TileInfo ti = decode_tile(d, t, gathered, rot0, rot1);
        const int nkb = (d.K[ti.prob] + BK - 1) / BK;
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, abort_flag)) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * kPairTileN;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&full_bar[s], phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * kPairStageBytes);
          const uint32_t b_addr = a_addr + kPairABytes;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = A_MN ? make_smem_desc_sw128(a_addr + k * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(a_addr + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc_sw128(b_addr + k * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(b_addr + k * 32, 16, 1024);
            tc_mma_bf16_pair(tmem_d, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          // the stage is free in both CTAs once these MMAs have read it
          const uint32_t e = smem_u32(&empty_bar[s]);
          tc_commit_pair(e);
          tc_commit_pair(mapa_u32(e, 1));
          if (++s == kPairStages) {
            s = 0;
            phase ^= 1u;
          }
        }
        if (ok) {
          const uint32_t f = smem_u32(&tfull_bar[acc]);
          tc_commit_pair(f);
          tc_commit_pair(mapa_u32(f, 1));
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (both CTAs)
    const int quarter = warp & 3;
    const int half = (warp - kEpiWarp0) >> 2;  // two warps per lane quarter, half of the columns each
    const int chunk0 = half * (kPairTileN / 64), chunk1 = chunk0 + kPairTileN / 64;
    int it = 0;
    for (int t = pair; t < total_tiles; t += npair, ++it) {
      const TileInfo ti = decode_tile(d, t, gathered, rot0, rot1);
      const Problem& p = args.p[ti.prob];
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag)) break;
      tc_fence_after();
      epilogue_rows<kPairTileN>(p, d.M[ti.prob], d.m0[ti.prob],
                                ti.mt * kPairTileM + static_cast<int>(rank) * BM + quarter * 32 + lane,
                                ti.nt * kPairTileN,
                                tmem_base + acc * kPairTileN + (static_cast<uint32_t>(quarter * 32) << 16), chunk0, chunk1);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (leader) mbar_arrive(&tempty_bar[acc]);
        else mbar_arrive_cluster(mapa_u32(smem_u32(&tempty_bar[acc]), 0));
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicExch(status, 1);
  cluster_arrive();  // nothing of the peer may still target this CTA's barriers or shared memory
  cluster_wait();
  if (warp == kEpiWarp0) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

// Co-resident CTA pairs of the device for this kernel (0 when clusters cannot be scheduled).
template <bool A_MN, bool B_MN>
int pair_capacity() {
  static int cap = -1;
  if (cap >= 0) return cap;
  auto kern = gemm_pair_kernel<A_MN, B_MN>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes) != cudaSuccess) {
    cudaGetLastError();
    return cap = 0;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * num_sms(), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = kPairSmemBytes;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  return cap = n;
}

template <bool A_MN, bool B_MN>
int launch_pair_t(const GemmArgs& args, long tiles, cudaStream_t stream, int* status) {
  const int cap = pair_capacity<A_MN, B_MN>();
  if (cap <= 0) return -10;
  const int pairs = tiles < cap ? static_cast<int>(tiles) : cap;
  gemm_pair_kernel<A_MN, B_MN><<<2 * pairs, kThreads, kPairSmemBytes, stream>>>(args, status);
  return static_cast<int>(cudaGetLastError());
}

// Gathered-weight launch on CTA pairs: `n_pull` copy CTAs (even) + GEMM pairs; -10 when clusters cannot be scheduled
// or too few pairs would be left.
template <bool A_MN, bool B_MN>
int launch_pair_ag_t(const GemmArgs& args, long tiles, int n_pull, cudaStream_t stream, int* status) {
  const int cap = pair_capacity<A_MN, B_MN>();  // same resources per CTA as the instantiation with copy CTAs
  if (cap <= n_pull / 2 + 1) return -10;
  auto kern = gemm_pair_kernel<A_MN, B_MN, true>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes) != cudaSuccess) {
      cudaGetLastError();
      return -10;
    }
    attr_set = true;
  }
  const int avail = cap - n_pull / 2;
  const int pairs = tiles < avail ? static_cast<int>(tiles) : avail;
  kern<<<n_pull + 2 * pairs, kThreads, kPairSmemBytes, stream>>>(args, status);
  return static_cast<int>(cudaGetLastError());
}

int launch_pair(const GemmArgs& args, bool a_mn, bool b_mn, long tiles, cudaStream_t stream, int* status) {
  if (!a_mn && !b_mn) return launch_pair_t<false, false>(args, tiles, stream, status);
  if (!a_mn && b_mn) return launch_pair_t<false, true>(args, tiles, stream, status);
  if (a_mn && !b_mn) return launch_pair_t<true, false>(args, tiles, stream, status);
  return launch_pair_t<true, true>(args, tiles, stream, status);
}

}  // namespace
}  // namespace wx
