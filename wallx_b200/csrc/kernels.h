// Host launchers of the non-GEMM kernels (raw pointers + stream; no torch types). Every function
// returns a CUDA error code (0 = ok) or a negative value for an unsupported shape.
// Reference parity: csrc/permute.cu:39-262 (permute / unpermute), csrc/rope.cu:48-330 (mRoPE), the unfused ATen
// RMSNorm of modeling_qwen2_5_vl.py:131-136, the SiLU * up product of modeling_qwen2_5_vl_act.py:79-82, the unreduced
// cross entropy of :1431-1444 and torch.optim.AdamW (wall_x/trainer/qwen_vl_act_trainer.py:577-581).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace wx {

int rms_norm_fwd(const void* x, const void* w, void* y, float* rstd, const int* dest, int T, int C, float eps,
                 cudaStream_t s);
int rms_norm_bwd_blocks(int T);
// `add` (optional, bf16 [T, C]): added to dx with the rounding of a separate bf16 add (the gradient that arrives
// over the residual connection around the normalised branch).
int rms_norm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const int* dest, void* dx,
                 float* dw_partial, void* dw, int T, int C, cudaStream_t s, const void* add = nullptr);
int swiglu_bwd(const void* dh, const void* gu, void* dgu, int R, int width_gu, long ld_dh, long ld_gu,
               cudaStream_t s);
// `out` may be `in` (in place: the columns that are not rotated are then left alone instead of copied).
int rope_qk(const void* in, void* out, const float* cos_t, const float* sin_t, int T, int W, int n_rot, int D,
            int inverse, cudaStream_t s);
int route_plan(const int* types, int T, int E, int rows, int* dest, int* seg, int* segk, int* inv, cudaStream_t s);
// `out_rows` / `src_rows` (0: unknown) are the row counts of the scattered-into / gathered-from buffer; only the
// range checks of the debug build read them.
int permute_rows(const void* x, const int* dest, void* out, int T, int C, cudaStream_t s, int out_rows = 0);
int gather_rows(const void* x, const int* idx, void* out, int T, int C, cudaStream_t s, int src_rows = 0);
// `partials`: fp32 scratch of column_sum_slabs(R) * C elements (need not be cleared)
int column_sum_slabs(int R);
int column_sum(const void* x, float* partials, void* out_bf16, int R, int C, cudaStream_t s);
int ce_fwd(const void* logits, const long* labels, float* loss, float* lse, long* pred, int R, int V, long ld,
           cudaStream_t s);
int ce_bwd(void* logits, const long* labels, const float* lse, const float* dloss, int R, int V, long ld,
           cudaStream_t s);
int sumsq_bf16(const void* g, long n, float* out, cudaStream_t s);
int adamw_step(void* p16, float* p32, float* m, float* v, const void* g, long n, const float* hyper,
               const float* norm_sq, cudaStream_t s);

// index generation (index.cu)
int rope_index(const long* ids, const int* mask, const int* img_grid, int n_img, const int* vid_grid, int n_vid,
               const float* sec_per_grid, int B, int S, int merge, long image_id, long video_id, long vstart_id,
               float tokens_per_second, long* pos, long* deltas, int* status, cudaStream_t s);
int vit_rot_pos(const float* inv_freq, int F, const int* grid, int G, int merge, float* out, long N, cudaStream_t s);
int vit_window_index(const int* grid, int G, int vw, int merge, long* window_index, int* cu_seqlens, cudaStream_t s);

// Debug build (-DWX_CHECK): {first violating site, violation count, two values} of each translation unit's range
// checks, cleared when `clear`; all zeros in a release build. Return a CUDA error code.
int kernels_check_read(long long* out4, int clear);
int index_check_read(long long* out4, int clear);

}  // namespace wx
