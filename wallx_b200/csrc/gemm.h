// Host API of the tcgen05 GEMM core (no torch types: raw pointers + a CUDA stream).
//
// One launch computes up to two independent problems ("dual asymmetric grouped GEMM": the two
// FFN experts have different row counts and different widths), each
//     D[m, n] = epilogue( sum_k A(m, k) * B(n, k) )
// with bf16 operands and fp32 accumulation in tensor memory.
//
// Parity: this covers the reference's csrc/dual_asym_grouped_gemm.cu:49-136 (NN/NT/TN/TT CUTLASS
// GemmGrouped for two problems) and every nn.Linear it runs through cuBLAS.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace wx {

enum GemmFlags : int {
  GEMM_OUT_FP32 = 1,     // D is fp32 (else bf16)
  GEMM_ACCUMULATE = 2,   // D += result (fp32 or bf16 read-modify-write)
  GEMM_ACT_GELU = 4,     // exact (erf) GELU after bias
  GEMM_ACT_SWIGLU = 8,   // B rows interleaved [16 gate | 16 up]: D[:, j] = silu(g_j) * u_j, ld = N/2
  GEMM_ZERO_PAD_ROWS = 16,  // rows in [M, round_up(M, 128)) are written as zeros (no row_map)
  // SwiGLU backward fused into the dgrad of the down projection: the accumulator is dL/dh [*, N];
  // D2 (input) holds the saved raw gate/up values [*, 2N] in 16-column interleaved blocks and D
  // (output, bf16, 2N wide) receives dL/d(gate|up) in the same layout. N % 32 == 0.
  GEMM_SWIGLU_BWD = 32,
};

struct GemmCall {
  // A(m, k): a_mn == false -> memory [a_rows][>=k0+K], k contiguous, pitch lda elements.
  //          a_mn == true  -> memory [k rows][a_rows'], m contiguous, pitch lda elements.
  const void* A;
  long lda;
  long a_extent_mn;  // number of valid m positions in memory (tensor-map bound along m)
  long a_extent_k;   // number of valid k positions in memory (tensor-map bound along k)
  bool a_mn;
  const void* B;
  long ldb;
  long b_extent_mn;
  long b_extent_k;
  bool b_mn;
  int M, N, K;
  int m0;  // offset along m applied to A coordinates and D rows
  int k0;  // offset along k applied to A and B coordinates
  // Optional device int[4] = {m0, M, k0, K}: non-negative entries override the static values
  // (data-dependent sizes without a host sync). The static M must then be an upper bound.
  const int* dyn;
  void* D;
  long ldd;
  long d_rows;  // rows of D in memory (0: unknown); only the range checks of the debug build read it
  void* D2;  // optional raw pre-activation output (bf16), SWIGLU only: [*, ldd2], N wide
  long ldd2;
  const void* bias;      // bf16 [N] or nullptr
  const void* residual;  // bf16 [*, ldr] added after activation, indexed by destination row
  long ldr;
  const int* row_map;  // optional: D row r is written to row row_map[r]; negative -> dropped
  int flags;
};

// Weight all-gather fused into the GEMM (ZeRO-3 style sharded weight): B's rows are split evenly
// over `world` ranks, rank r holding rows [r * rows_per_rank, (r + 1) * rows_per_rank) at
// peer[r] (peer-mapped memory over NVLink). A few CTAs of the persistent grid pull the shards
// into `staging` (this GPU's memory, [N][K]) one 256-row tile at a time with bulk copies and
// publish a flag per tile; the GEMM CTAs take the tiles in the same order and wait (bounded) on
// the flag before loading a B tile from `staging` by TMA. No load uses cluster multicast.
struct AgInfo {
  const void* peer[8];  // peer[r]: rank r's shard, [rows_per_rank][K] bf16, pitch K
  void* staging;        // this GPU's [N][K] bf16 buffer that the GEMM reads B from
  int* flags;           // device int[ceil(N / 256)]; every puller adds 1 per tile per call
  int world, rank, rows_per_rank;
  int n_pullers;        // CTAs of the grid that copy instead of multiplying (0 = default)
  int epoch;            // 1, 2, 3, ... per call on the same flags; a tile is ready at n_pullers * epoch
};

// Launches on `stream`. `status` is a device int that the kernel sets non-zero when one of its
// bounded waits ran out (the kernel then returns normally). Returns a CUDA error code (0 = ok).
int gemm_launch(const GemmCall* calls, int ncalls, cudaStream_t stream, int* status, int force_bn);

// One or two problems (A K-major; B K-major for the forward, MN-major for dgrad) whose B operand, the
// weight [N][K] resp. [K][N], is gathered from `ag.peer` while the GEMM runs; call.B must be
// ag.staging and call.ldb the weight's row length. Tile width is fixed at 256. Every rank's
// shard must be complete before any rank launches (a barrier between the optimizer step and the
// first gather is the caller's job).
int gemm_ag_launch(const GemmCall* calls, const AgInfo* ags, int ncalls, cudaStream_t stream, int* status);

// One or two problems whose operands are all in place, plus up to two weight gathers (ags[i] with row length cols[i])
// that the launch's copy CTAs run for later launches; nothing in this launch waits for them. See gemm.cu.
int gemm_launch_prefetch(const GemmCall* calls, int ncalls, const AgInfo* ags, const long* cols, int n_ags, cudaStream_t stream,
                         int* status);

// Rates (TFLOP/s) that steer the tile choice of gemm_launch: 128 x 256 / 128 x 128 / 128 x 64 single-CTA tiles and the
// 256 x 256 CTA-pair tile. Start-up values are one B200's; a caller may replace them with what it measured on the
// device in use (non-positive entries are ignored).
void gemm_set_tile_rates(const double* rates4);
void gemm_get_tile_rates(double* rates4);

// Debug build (-DWX_CHECK): copies out {first violating site, violation count, two values} of this translation
// unit's range checks and clears the record when `clear`; all zeros in a release build. Returns a CUDA error code.
int gemm_check_read(long long* out4, int clear);
int gemm_checked_build();  // 1 when the kernels were compiled with -DWX_CHECK

}  // namespace wx
