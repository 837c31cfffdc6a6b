// Host API of the tcgen05 varlen attention kernels (raw pointers + stream).
// Reference parity: flash-attn 2 behind wall_x/model/qwen2_5_based/modeling_qwen2_5_vl.py:208-210 (ViT, varlen,
// non-causal) and :1008-1015 (LLM, causal, GQA), plus the bidirectional action block of the mask builder in
// modeling_qwen2_5_vl_act.py:276-732.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace wx {

struct AttnShape {
  int Tq, Tk, hq, hkv, D;
  long ld_q, ld_k, ld_v;  // row pitch in elements of the q / k / v views
  float scale;
  int has_bidir;    // some query carries the bidirectional flag
  int causal_self;  // self-attention, causal, no bidirectional block: lets dK/dV skip query blocks
};

// qtab: int32 [Tq, 4] = (k_lo, k_hi, k_lim, flag); ktab: int32 [Tk, 4] = (q_lo, q_hi, q_causal, flag | q_first << 1):
// q_causal = first query row that sees the key under the causal rule (q_lo when not causal),
// q_first = first query row that sees it at all (lets dK/dV skip earlier query blocks).
// lse: fp32 [hq, Tq] (natural log). `status` is set non-zero when a bounded wait ran out.
int attn_fwd(const AttnShape& s, const void* q, const void* k, const void* v, const void* qtab, const void* ktab,
             void* out, long ld_out, float* lse, cudaStream_t stream, int* status);

// delta: fp32 scratch [hq, Tq]; part_k / part_v: fp32 scratch [hq/hkv, Tk, hkv*D], needed only
// when hq != hkv (partial dK/dV per query head of a group, summed at the end).
int attn_bwd(const AttnShape& s, const void* q, const void* k, const void* v, const void* out, long ld_o,
             const void* dout, long ld_do, const float* lse, const void* qtab, const void* ktab, float* delta,
             void* dq, long ld_dq, void* dk, long ld_dk, void* dv, long ld_dv, float* part_k, float* part_v,
             cudaStream_t stream, int* status);

// Debug build (-DWX_CHECK): this translation unit's range-check record {first violating site, violation count, two
// values}, cleared when `clear`; all zeros in a release build. Returns a CUDA error code.
int attn_check_read(long long* out4, int clear);

}  // namespace wx
