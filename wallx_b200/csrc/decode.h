// Host launchers of the cached decode / denoise step kernels (decode.cu): raw pointers + stream, CUDA error code or a
// negative value for an unsupported shape.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace wx {

// Rotary on the q and k heads of `qkv` [T, (hq + 2 hkv) D] (q rotated in place); the rotated k and the v columns of
// row t are written to row `cache_rows[t]` of `cache` ([cache_nrows, ld_cache], k then v).
int rope_cache(void* qkv, const float* cos_t, const float* sin_t, const long* cache_rows, void* cache, int T, int W,
               int hq, int hkv, int D, long ld_cache, long cache_nrows, cudaStream_t s);

// Attention of Tq <= 256 query rows over cached keys / values; `qtab` / `ktab` are the per-row tables of the
// tensor-core attention kernel (int4 per query row: first key, end key, causal limit, flag; int4 per key row: bit 0 of
// .w = flagged key). `max_keys`: the longest key range of a query row (0: unknown), which sets how many CTAs share a row.
bool attn_decode_supported(int Tq, int hq, int hkv, int D);
int attn_decode(const void* q, long ldq, const void* k, long ldk, const void* v, long ldv, const void* qtab,
                const void* ktab, void* out, long ldo, int Tq, int Tk, int hq, int hkv, int D, float scale, int max_keys,
                cudaStream_t s);

int decode_check_read(long long* out4, int clear);

}  // namespace wx
