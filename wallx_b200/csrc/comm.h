// Peer-memory collectives for the sharded optimizer (raw pointers + stream). All kernels read or
// write other GPUs' memory through plain peer pointers over NVLink / NVSwitch; no NCCL call.
// Reference parity: the NCCL reduce-scatter / all-gather that torch FSDP2 issues for the reference trainer
// (train_qact.py:42-49, wall_x/trainer/qwen_vl_act_trainer.py:609-611), its clip_grad_norm_ all-reduce (:335-337)
// and the per-step scalar gathers (:352-423).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace wx {

constexpr int kMaxPeers = 8;

struct PeerPtrs {
  void* p[kMaxPeers];
};

// Table entry: one flat buffer's shard. `arena_off` is the element offset of this rank's shard in
// every rank's bf16 arena, `n` its length, `out_off` the offset in the local fp32 shard buffer.
struct ShardDesc {
  long arena_off;
  long n;
  long out_off;
};

// Every rank signals every peer and waits (bounded) until all peers signalled `epoch`.
// flags.p[r] points at rank r's int[kMaxPeers] flag array. Sets *status non-zero on time-out
// (`timeout_ms`, clamped to [1 ms, 10 min]: training barriers must tolerate a rank that is late by a
// data-loader hiccup, failure tests want a short limit).
int symm_barrier(const PeerPtrs& flags, int rank, int world, int epoch, int* status, cudaStream_t s,
                 long timeout_ms = 2000);

// out[out_off + i] = sum_r bf16(grads.p[r][arena_off + i]) in fp32, for every table entry; adds the
// sum of squares of the results into *sumsq.
int rs_reduce(const PeerPtrs& grads, const ShardDesc* table_dev, int nbuf, int world, float* out, float* sumsq,
              cudaStream_t s);

// Copies this rank's bf16 shards (table entries) from its own arena into every peer's arena.
int ag_push(const PeerPtrs& params, const ShardDesc* table_dev, int nbuf, int rank, int world, cudaStream_t s);

// The same copy through an NVSwitch multicast mapping of the arena (`mc_base`, from the symmetric-memory rendezvous):
// multimem.st makes the switch replicate every 16 bytes into all GPUs' arenas, so the shard leaves this GPU once.
// A barrier must follow before anyone reads the parameters, as for ag_push.
int ag_push_multicast(void* mc_base, const void* local_base, const ShardDesc* table_dev, int nbuf, cudaStream_t s);

// All-reduce (sum) of a small fp32 vector: each rank writes its values into slot `rank` of every
// peer's scratch [world][n]; after the barrier every rank sums the `world` slots into out.
int small_allreduce_write(const PeerPtrs& scratch, const float* vals, int n, int rank, int world, cudaStream_t s);
int small_allreduce_sum(const float* my_scratch, float* out, int n, int world, cudaStream_t s);

// AdamW on fp32 gradients (see adamw_step in kernels.h for the hyper-parameter layout).
int adamw_step_f32g(void* p16, float* p32, float* m, float* v, const float* g, long n, const float* hyper,
                    const float* norm_sq, cudaStream_t s);

// Debug build (-DWX_CHECK): this translation unit's range-check record (see kernels.h); zeros in a release build.
int comm_check_read(long long* out4, int clear);

}  // namespace wx
