// Few-row GEMM for sm_100a: out[M <= 128, N] = A[M, K] . W[N, K]^T, both operands K-major (decode and denoise steps:
// 32 action rows against every weight of a layer). Included by gemm.cu after the general kernel.
//
// What limits such a product is neither the tensor pipe nor DRAM but the serial chain inside one CTA: measured on a
// B200, a CTA of the general kernel (or of a one-CTA-per-column-tile variant of it) spends about 0.3 us per 64-wide
// k block (wait for the stage, four tcgen05.mma whose 128-row A operand is read from shared memory whatever the row
// count, commit), i.e. 10 us for K = 2048 with every unit of the GPU idle. So the work is cut along K as well:
//   * one *cluster* of `splits` CTAs per 64 output columns, CTA r of the cluster owning the k blocks
//     [nkb * r / splits, nkb * (r + 1) / splits) -- 2048 x 2048 runs as 32 clusters of 4, eight k blocks per CTA;
//   * a stage holds only the rows that exist (32, 64 or 128) and a 64-row slice of the weight; with so few k blocks
//     per CTA all of its loads are in flight at once and a stage is handed back only if the ring actually wraps;
//   * every CTA leaves its fp32 partial tile in its own shared memory; after a cluster barrier the (row, 32-column)
//     pieces of the tile are dealt round-robin to the threads of all CTAs of the cluster, which add the partials in
//     rank order through distributed shared memory (a fixed order: results do not depend on timing) and run the
//     usual epilogue (bias / SwiGLU / residual / fp32 / accumulate / row map).
// tcgen05.mma runs at M = 128 whatever the row count: the A descriptor reaches past the loaded rows into the bytes
// that follow in shared memory (the B slice, later stages, a slack area after the last stage). Those accumulator
// rows hold garbage, stay in their own TMEM lanes and are never stored. With one split the sum over K has the order
// of the general kernel (bit-identical results); with more it is a sum of per-split partial sums.
#pragma once

namespace wx {
namespace {

constexpr int kSkinnyBN = 64;
constexpr int kSkinnyThreads = 192;  // TMA warp, MMA warp, 4 epilogue warps (one per TMEM lane quarter)
constexpr int kMidBN = 256;    // tile width of the same kernel for 129..1024 rows (128-row tiles, see gemm_launch)
constexpr int kSkinnyMaxSplits = 8;          // portable cluster size

__device__ __forceinline__ void prefetch_l1(const void* p) { asm volatile("prefetch.global.L1 [%0];" ::"l"(p)); }

template <int A_ROWS, int BN>
struct SkinnyCfg {
  static constexpr int A_BYTES = A_ROWS * BK * 2;
  static constexpr int PITCH = BN + 4;  // floats per row of the partial tile (16-byte row stores without conflicts)
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // about 100 KB of stages, so that two CTAs fit on an SM: under programmatic dependent launch the CTAs of the next
  // few-row GEMM then sit beside this one's and stream their weights while this one finishes
  static constexpr int STAGES = (BN == 256) ? 4 : (A_ROWS == 32) ? 8 : (A_ROWS == 64) ? 6 : 4;
  static constexpr int SLACK = BM * BK * 2 - A_BYTES;  // what the 128-row A descriptor reads beyond the last stage's rows
  static constexpr int PARTIAL_BYTES = A_ROWS * PITCH * 4;  // aliases the start of the ring once the MMAs are done
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + SLACK + 1024 + 512;
  static_assert(SMEM_BYTES <= 227 * 1024, "stage ring does not fit");
  static_assert(STAGE_BYTES % 1024 == 0, "stages must keep the 1024-byte alignment of the swizzle pattern");
  static_assert(PARTIAL_BYTES <= STAGES * STAGE_BYTES, "partial tile must fit in the ring");
};

template <int A_ROWS, int BN>
__global__ void __launch_bounds__(kSkinnyThreads, 1)
gemm_skinny_kernel(const __grid_constant__ GemmArgs args, int* __restrict__ status, int splits) {
  using C = SkinnyCfg<A_ROWS, BN>;
  // Clusters are laid out from the static sizes (problem 0's column tiles, then problem 1's); the row count and K
  // may be smaller on the device (dyn). Everything that decides whether a CTA works is uniform over its cluster.
  const int tile = static_cast<int>(blockIdx.x) / splits;
  const int rank = static_cast<int>(blockIdx.x) - tile * splits;  // = %cluster_ctarank
  // tiles of a problem: column tiles x 128-row tiles (static row count), row tiles fastest so that the clusters
  // which share a weight slice run at the same time
  const int mt0 = (args.p[0].M + BM - 1) / BM;
  const int t0 = ((args.p[0].N + BN - 1) / BN) * mt0;
  const int prob = tile < t0 ? 0 : 1;
  const int mtiles = prob ? (args.p[1].M + BM - 1) / BM : mt0;
  const int tp = tile - (prob ? t0 : 0);
  const int nt = tp / mtiles;
  const int mt = tp - nt * mtiles;
  if (prob >= args.nprob) return;  // cannot happen with the host's grid
  const Problem& p = args.p[prob];

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES + C::SLACK);
  uint64_t* empty_bar = full_bar + C::STAGES;
  uint64_t* tfull_bar = empty_bar + C::STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tfull_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* partial = reinterpret_cast<float*>(smem);

  // ---- prologue: nothing here reads memory that an earlier kernel writes, so under programmatic dependent launch it
  // runs while the kernel ahead in the stream is still finishing
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // With static sizes (no device-side row count or K) the weight loads depend on nothing an earlier kernel writes:
  // they are issued here, ahead of the wait on that kernel; the activation loads follow the wait.
  const int tile_n = nt * BN;
  int early = 0;
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tfull_bar, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&p.tmA);
    tma_prefetch_desc(&p.tmB);
    if (p.dyn == nullptr && p.M > mt * BM && p.K > 0 && (p.k0 & 7) == 0 && tile_n < p.N) {
      const int nkb_s = (p.K + BK - 1) / BK;
      const int b0 = static_cast<int>(static_cast<long>(nkb_s) * rank / splits);
      const int b1 = static_cast<int>(static_cast<long>(nkb_s) * (rank + 1) / splits);
      early = min(b1 - b0, C::STAGES);
      for (int j = 0; j < early; ++j) {
        mbar_arrive_expect_tx(&full_bar[j], C::STAGE_BYTES);
        tma_load_2d(smem + j * C::STAGE_BYTES + C::A_BYTES, &p.tmB, &full_bar[j], p.k0 + (b0 + j) * BK, tile_n);
      }
    }
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();
  pdl_launch_dependents();

  int M = p.M, K = p.K, m0 = p.m0, k0 = p.k0;
  if (p.dyn != nullptr) {
    const int d0 = p.dyn[0], d1 = p.dyn[1], d2 = p.dyn[2], d3 = p.dyn[3];
    if (d0 >= 0) m0 = d0;
    if (d1 >= 0) M = min(d1, p.M);
    if (d2 >= 0) k0 = d2;
    if (d3 >= 0) K = d3;
  }
  // a problem without rows on the device, or a column tile past N: nothing to do (uniform over the cluster)
  M -= mt * BM;  // rows of this tile (the last row tile of a problem may be short, or empty on the device)
  m0 += mt * BM;
  if (M > BM) M = BM;
  const bool live = M > 0 && K > 0 && nt * BN < p.N && WX_CHK(M <= A_ROWS && (k0 & 7) == 0, 2006, M, k0);

  const int nkb = (K + BK - 1) / BK;
  const int kb0 = static_cast<int>(static_cast<long>(nkb) * rank / splits);
  const int kb1 = static_cast<int>(static_cast<long>(nkb) * (rank + 1) / splits);
  const int nblk = kb1 - kb0;  // this CTA's k blocks (0 when there are more CTAs than blocks: it contributes zeros)
  const int n_base = nt * BN;

  if (!live) {
    // straight to the teardown: no cluster barrier is used by a cluster that does not work
  } else {
    if (warp == 0) {
      if (lane == 0) {
        for (int j = 0; j < nblk; ++j) {
          const int s = j % C::STAGES;
          const int use = j / C::STAGES;
          if (use > 0 && !mbar_wait(&empty_bar[s], static_cast<uint32_t>(use - 1) & 1u, abort_flag)) break;
          uint8_t* sA = smem + s * C::STAGE_BYTES;
          const int kc = k0 + (kb0 + j) * BK;
          if (j >= early) {  // (the first `early` weight slices are already on their way)
            mbar_arrive_expect_tx(&full_bar[s], C::STAGE_BYTES);
            tma_load_2d(sA + C::A_BYTES, &p.tmB, &full_bar[s], kc, n_base);  // the weight slice first: it comes from DRAM
          }
          tma_load_2d(sA, &p.tmA, &full_bar[s], kc, m0);
        }
      }
    } else if (warp == 1) {
      if (lane == 0) {
        constexpr uint32_t idesc = make_idesc_bf16(BM, BN, false, false);
        bool ok = true;
        for (int j = 0; j < nblk; ++j) {
          const int s = j % C::STAGES;
          const int use = j / C::STAGES;
          if (!mbar_wait(&full_bar[s], static_cast<uint32_t>(use) & 1u, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * C::STAGE_BYTES);
          const uint32_t b_addr = a_addr + C::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            tc_mma_bf16(tmem_base, make_smem_desc_sw128(a_addr + k * 32, 16, 1024),
                        make_smem_desc_sw128(b_addr + k * 32, 16, 1024), idesc, (j | k) != 0 ? 1u : 0u);
          if (j + C::STAGES < nblk) tc_commit(&empty_bar[s]);  // only a stage that will be loaded again is handed back
        }
        if (ok && nblk > 0) tc_commit(tfull_bar);
      }
    } else {
      // ---- this CTA's partial tile: tensor memory -> shared memory (rows of this warp's lane quarter)
      const int quarter = warp & 3;
      if (quarter * 32 < A_ROWS && quarter * 32 < M) {
        bool have = nblk > 0;
        if (have) {
          have = mbar_wait(tfull_bar, 0u, abort_flag);
          tc_fence_after();
        }
        float* prow = partial + (quarter * 32 + lane) * C::PITCH;
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          if (have) {
            tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + c * 32, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = 0u;
          }
#pragma unroll
          for (int q4 = 0; q4 < 8; ++q4)
            *reinterpret_cast<uint4*>(prow + c * 32 + 4 * q4) = make_uint4(r[4 * q4], r[4 * q4 + 1], r[4 * q4 + 2], r[4 * q4 + 3]);
        }
        tc_fence_before();
      }
    }
    // What the epilogue of this thread's first piece will read from global memory (row map, residual, bias) is
    // requested now, so that it arrives while the cluster barrier is being waited for.
    const int pieces = M * (BN / 32);
    {
      const int i = static_cast<int>(threadIdx.x) * splits + rank;
      if (i < pieces) {
        const int r = i / (BN / 32);
        const int n0 = n_base + (i - r * (BN / 32)) * 32;
        long drow = static_cast<long>(m0) + r;
        if (p.row_map != nullptr) drow = p.row_map[drow];
        if (drow >= 0 && n0 < p.N) {
          if (p.residual != nullptr) prefetch_l1(p.residual + drow * p.ldr + n0);
          if (p.bias != nullptr) prefetch_l1(p.bias + n0);
        }
      }
    }
    // (the tile overwrites the first stages: every MMA that read them has completed, tfull_bar says so)
    __syncthreads();
    if (splits > 1) {
      cluster_arrive();
      cluster_wait();
    }
    // ---- sum over the cluster and epilogue: piece i = (row i / 2, 32-column half i % 2) goes to CTA i % splits
    const uint32_t partial_addr = smem_u32(partial);
    for (int slot = threadIdx.x;; slot += kSkinnyThreads) {
      const int i = slot * splits + rank;
      if (i >= pieces) break;
      const int r = i / (BN / 32);
      const int c = i - r * (BN / 32);
      const int n0 = n_base + c * 32;
      if (n0 >= p.N) continue;
      float v[32];
#pragma unroll
      for (int e = 0; e < 32; ++e) v[e] = 0.f;
      const uint32_t off = static_cast<uint32_t>((r * C::PITCH + c * 32) * 4);
      // two CTAs' pieces are requested before either is added (16 loads in flight); the sums keep the rank order
      for (int s = 0; s < splits; s += 2) {
        const bool two = s + 1 < splits;
        const uint32_t base0 = mapa_u32(partial_addr + off, static_cast<uint32_t>(s));
        const uint32_t base1 = mapa_u32(partial_addr + off, static_cast<uint32_t>(two ? s + 1 : s));
        float4 x0[8], x1[8];
#pragma unroll
        for (int q4 = 0; q4 < 8; ++q4) x0[q4] = ld_cluster_f32x4(base0 + 16 * q4);
#pragma unroll
        for (int q4 = 0; q4 < 8; ++q4) x1[q4] = two ? ld_cluster_f32x4(base1 + 16 * q4) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int q4 = 0; q4 < 8; ++q4) {
          v[4 * q4] += x0[q4].x;
          v[4 * q4 + 1] += x0[q4].y;
          v[4 * q4 + 2] += x0[q4].z;
          v[4 * q4 + 3] += x0[q4].w;
        }
        if (two) {
#pragma unroll
          for (int q4 = 0; q4 < 8; ++q4) {
            v[4 * q4] += x1[q4].x;
            v[4 * q4 + 1] += x1[q4].y;
            v[4 * q4 + 2] += x1[q4].z;
            v[4 * q4 + 3] += x1[q4].w;
          }
        }
      }
      long drow = static_cast<long>(m0) + r;
      if (p.row_map != nullptr) {
        const int mapped = p.row_map[drow];
        if (mapped < 0) continue;
        drow = mapped;
      }
      if (!WX_CHK(drow >= 0 && (p.d_rows == 0 || drow < p.d_rows), 2007, drow, p.d_rows)) continue;
      epilogue_chunk(p, v, drow, n0, false);
    }
    __syncthreads();
    if (splits > 1) {  // nobody leaves while a peer may still read its tile
      cluster_arrive();
      cluster_wait();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicExch(status, 1);
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, BN);
  }
}

template <int A_ROWS, int BN>
int launch_skinny_t(const GemmArgs& args, int tiles, int splits, cudaStream_t stream, int* status) {
  using C = SkinnyCfg<A_ROWS, BN>;
  auto kern = gemm_skinny_kernel<A_ROWS, BN>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set = true;
  }
  return static_cast<int>(launch_kernel_cluster(kern, dim3(static_cast<unsigned>(tiles * splits)), dim3(kSkinnyThreads),
                                                C::SMEM_BYTES, stream, static_cast<unsigned>(splits), args, status, splits));
}

// Rows staged per k step for a launch whose largest problem has `max_m` rows.
inline int skinny_rows(int max_m) { return max_m <= 32 ? 32 : max_m <= 64 ? 64 : 128; }

// CTAs per cluster: as many as keep all clusters in one wave (a power of two, at most 8), each with two k blocks or more.
inline int skinny_splits(long tiles, int min_nkb, int sms) {
  int s = 1;
  while (s * 2 <= kSkinnyMaxSplits && tiles * (s * 2) <= sms && min_nkb >= 2 * (s * 2)) s *= 2;
  return s;
}

int launch_skinny(const GemmArgs& args, int a_rows, int bn, int tiles, int splits, cudaStream_t stream, int* status) {
  if (bn == kMidBN) return launch_skinny_t<128, kMidBN>(args, tiles, splits, stream, status);
  if (a_rows == 32) return launch_skinny_t<32, kSkinnyBN>(args, tiles, splits, stream, status);
  if (a_rows == 64) return launch_skinny_t<64, kSkinnyBN>(args, tiles, splits, stream, status);
  return launch_skinny_t<128, kSkinnyBN>(args, tiles, splits, stream, status);
}

}  // namespace
}  // namespace wx
