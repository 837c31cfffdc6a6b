// Index-generation kernels (latency-bound, one launch each, exact integer arithmetic, no host
// round trips): LLM 3-axis rope positions, ViT rotary angle table, ViT window permutation.
//
// Reference parity: csrc/rope_index.cu (three kernels, float-reciprocal division, at most 64 vision
// items per sample), csrc/rot_pos.cu (two kernels on the legacy default stream + two device
// syncs), csrc/window_index.cu (four kernels, two D2H copies, a cross-block scan race); Python
// originals modeling_qwen2_5_vl_act.py:929-1149 and modeling_qwen2_5_vl.py:473-547.
#include "kernels.h"
#include "check.cuh"

namespace wx {

namespace {

constexpr int RI_THREADS = 256;
constexpr int RI_MAX_ITEMS = 512;

struct VisionItem {
  int start;       // compact index of the first vision token
  int n;           // number of vision tokens (t * gh * gw)
  int gh, gw;
  int base;        // position of the item's origin (text before it included)
  float tsec;      // seconds per temporal grid step * tokens_per_second (0 for images)
  int text_start;  // compact index where the text run before the item starts
  int text_base;   // position of that text run's first token
};

// One block per sample. Shared memory: int tok[S] | int cpos[S] (compact index -> original column).
__global__ void __launch_bounds__(RI_THREADS)
rope_index_kernel(const long* __restrict__ ids, const int* __restrict__ mask, const int* __restrict__ img_grid, int n_img,
                  const int* __restrict__ vid_grid, int n_vid, const float* __restrict__ sec_per_grid, int B, int S,
                  int merge, long image_id, long video_id, long vstart_id, float tokens_per_second,
                  long* __restrict__ pos, long* __restrict__ deltas, int* __restrict__ status) {
  extern __shared__ int sm[];
  int* tok = sm;
  int* cpos = sm + S;
  __shared__ VisionItem items[RI_MAX_ITEMS];
  __shared__ int s_nvalid, s_nitems, s_img0, s_vid0, s_tail_start, s_tail_base, s_max;
  __shared__ int s_scan[RI_THREADS];
  const int b = blockIdx.x, tid = threadIdx.x;

  // ---- images / videos consumed by earlier samples (vision-start followed by the media token)
  int ci = 0, cv = 0;
  for (long i = tid; i < static_cast<long>(b) * S; i += RI_THREADS) {
    const int col = static_cast<int>(i % S);
    if (col + 1 >= S) continue;
    if (mask != nullptr && (mask[i] == 0 || mask[i + 1] == 0)) continue;
    if (ids[i] == vstart_id) {
      ci += ids[i + 1] == image_id;
      cv += ids[i + 1] == video_id;
    }
  }
  if (tid == 0) {
    s_img0 = 0;
    s_vid0 = 0;
    s_max = 0;
  }
  __syncthreads();
  if (ci) atomicAdd(&s_img0, ci);
  if (cv) atomicAdd(&s_vid0, cv);

  // ---- compact the valid tokens of this sample (block-wide prefix count over the mask)
  int run = 0;
  for (int base = 0; base < S; base += RI_THREADS) {
    const int s = base + tid;
    const int v = (s < S) ? (mask == nullptr ? 1 : (mask[static_cast<long>(b) * S + s] != 0)) : 0;
    s_scan[tid] = v;
    __syncthreads();
    for (int off = 1; off < RI_THREADS; off <<= 1) {
      const int add = (tid >= off) ? s_scan[tid - off] : 0;
      __syncthreads();
      s_scan[tid] += add;
      __syncthreads();
    }
    if (v) {
      const int c = run + s_scan[tid] - 1;
      tok[c] = static_cast<int>(ids[static_cast<long>(b) * S + s]);
      cpos[c] = s;
    }
    run += s_scan[RI_THREADS - 1];
    __syncthreads();
  }
  if (tid == 0) s_nvalid = run;
  __syncthreads();
  const int n = s_nvalid;

  // ---- walk the vision items in order of appearance (serial: a handful per sample)
  if (tid == 0) {
    int rem_i = 0, rem_v = 0;
    for (int i = 0; i + 1 < n; ++i)
      if (tok[i] == static_cast<int>(vstart_id)) {
        rem_i += tok[i + 1] == static_cast<int>(image_id);
        rem_v += tok[i + 1] == static_cast<int>(video_id);
      }
    int ii = s_img0, vi = s_vid0, st = 0, nxt = 0, k = 0;
    const int total = rem_i + rem_v;
    for (int it = 0; it < total; ++it) {
      int ed_i = n + 1, ed_v = n + 1;
      if (rem_i > 0)
        for (int i = st; i < n; ++i)
          if (tok[i] == static_cast<int>(image_id)) {
            ed_i = i;
            break;
          }
      if (rem_v > 0)
        for (int i = st; i < n; ++i)
          if (tok[i] == static_cast<int>(video_id)) {
            ed_v = i;
            break;
          }
      int t, h, w, ed;
      float sec = 0.f;
      if (ed_i < ed_v) {
        if (ii >= n_img) break;
        t = img_grid[ii * 3];
        h = img_grid[ii * 3 + 1];
        w = img_grid[ii * 3 + 2];
        ++ii;
        --rem_i;
        ed = ed_i;
      } else {
        if (vi >= n_vid || ed_v > n) break;
        t = vid_grid[vi * 3];
        h = vid_grid[vi * 3 + 1];
        w = vid_grid[vi * 3 + 2];
        sec = (sec_per_grid ? sec_per_grid[vi] : 1.0f) * tokens_per_second;
        ++vi;
        --rem_v;
        ed = ed_v;
      }
      if (k >= RI_MAX_ITEMS) {
        atomicExch(status, 32);  // more vision items in one sample than the kernel holds
        break;
      }
      const int gh = h / merge, gw = w / merge;
      VisionItem v;
      v.text_start = st;
      v.text_base = nxt;
      v.start = ed;
      v.n = t * gh * gw;
      v.gh = gh;
      v.gw = gw;
      v.base = nxt + (ed - st);
      v.tsec = sec;
      items[k++] = v;
      const int tmax = static_cast<int>(static_cast<float>(t - 1) * sec);
      nxt = v.base + max(tmax, max(gh - 1, gw - 1)) + 1;
      st = ed + v.n;
    }
    s_nitems = k;
    s_tail_start = st;
    s_tail_base = nxt;
  }
  __syncthreads();

  // ---- positions, one thread per column
  const int nitems = s_nitems;
  const long plane = static_cast<long>(B) * S;
  long* p0 = pos + static_cast<long>(b) * S;
  for (int s = tid; s < S; s += RI_THREADS) {
    p0[s] = 1;
    p0[plane + s] = 1;
    p0[2 * plane + s] = 1;
  }
  __syncthreads();
  int local_max = 0;
  for (int c = tid; c < n; c += RI_THREADS) {
    int pt, ph, pw;
    if (c >= s_tail_start) {
      pt = ph = pw = s_tail_base + (c - s_tail_start);
    } else {
      int k = 0;
      while (k + 1 < nitems && c >= items[k + 1].text_start) ++k;
      const VisionItem v = items[k];
      if (c < v.start) {
        pt = ph = pw = v.text_base + (c - v.text_start);
      } else {
        const int o = c - v.start;
        const int hw = v.gh * v.gw;
        const int ti = o / hw, r = o - ti * hw;
        const int hi = r / v.gw, wi = r - hi * v.gw;
        pt = v.base + static_cast<int>(static_cast<float>(ti) * v.tsec);
        ph = v.base + hi;
        pw = v.base + wi;
      }
    }
    const int s = cpos[c];
    if (!WX_CHK(s >= 0 && s < S, 5001, s, S)) continue;
    p0[s] = pt;
    p0[plane + s] = ph;
    p0[2 * plane + s] = pw;
    local_max = max(local_max, max(pt, max(ph, pw)));
  }
  atomicMax(&s_max, local_max);
  __syncthreads();
  if (tid == 0) deltas[b] = (n > 0) ? static_cast<long>(s_max) + 1 - S : 0;
}

// ------------------------------------------------------------------------------ ViT rotary angles
__global__ void vit_rot_pos_kernel(const float* __restrict__ inv_freq, int F, const int* __restrict__ grid, int G,
                                   int merge, float* __restrict__ out, long N) {
  const long idx = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= N * F) return;
  const long patch = idx / F;
  const int f = static_cast<int>(idx - patch * F);
  long off = 0;
  int g = 0, t = 1, h = 1, w = 1;
  for (; g < G; ++g) {
    t = grid[g * 3];
    h = grid[g * 3 + 1];
    w = grid[g * 3 + 2];
    const long cnt = static_cast<long>(t) * h * w;
    if (patch < off + cnt) break;
    off += cnt;
  }
  if (g >= G) return;
  const int l = static_cast<int>(patch - off);
  const int hw = h * w;
  const int r = l % hw;
  const int mm = merge * merge;
  const int bi = r / mm, within = r - bi * mm;
  const int bw = w / merge;
  const int brow = bi / bw, bcol = bi - brow * bw;
  const int hpos = brow * merge + within / merge;
  const int wpos = bcol * merge + within % merge;
  const float fr = inv_freq[f];
  if (!WX_CHK(patch >= 0 && patch < N && hpos >= 0 && hpos < h && wpos >= 0 && wpos < w, 5002, patch, hpos)) return;
  out[patch * (2 * F) + f] = static_cast<float>(hpos) * fr;
  out[patch * (2 * F) + F + f] = static_cast<float>(wpos) * fr;
}

// ------------------------------------------------------------------------------ ViT window index
// One block per image/video grid. Windows are numbered (frame, window row, window column); the
// reference's padding rule adds a full extra row/column of windows when the size is a multiple of
// the window (those windows are empty and repeat the previous offset in cu_window_seqlens).
__global__ void __launch_bounds__(256)
vit_window_index_kernel(const int* __restrict__ grid, int G, int vw, int merge, long* __restrict__ window_index,
                        int* __restrict__ cu_seqlens) {
  __shared__ long s_tok_base;
  __shared__ int s_win_base;
  const int g = blockIdx.x, tid = threadIdx.x;
  if (tid == 0) {
    long tb = 0;
    int wb = 0;
    for (int i = 0; i < g; ++i) {
      const int t = grid[i * 3], gh = grid[i * 3 + 1] / merge, gw = grid[i * 3 + 2] / merge;
      tb += static_cast<long>(t) * gh * gw;
      wb += t * ((gh + vw - gh % vw) / vw) * ((gw + vw - gw % vw) / vw);
    }
    s_tok_base = tb;
    s_win_base = wb;
    if (g == 0) cu_seqlens[0] = 0;
  }
  __syncthreads();
  const int t = grid[g * 3], gh = grid[g * 3 + 1] / merge, gw = grid[g * 3 + 2] / merge;
  const int nh = (gh + vw - gh % vw) / vw, nw = (gw + vw - gw % vw) / vw;
  const int unit = merge * merge;
  const int nwin = t * nh * nw;
  // tokens before window k of this grid, closed form: full frames, full window rows, then columns
  for (int k = tid; k < nwin; k += blockDim.x) {
    const int ti = k / (nh * nw), r = k - ti * nh * nw;
    const int wr = r / nw, wc = r - wr * nw;
    const int rows = max(0, min(vw, gh - wr * vw));
    const int cols = max(0, min(vw, gw - wc * vw));
    const int rows_before = min(gh, wr * vw);
    const int cols_before = min(gw, wc * vw);
    const long excl = static_cast<long>(ti) * gh * gw + static_cast<long>(rows_before) * gw +
                      static_cast<long>(rows) * cols_before;
    cu_seqlens[s_win_base + k + 1] = static_cast<int>((s_tok_base + excl + static_cast<long>(rows) * cols) * unit);
    for (int e = 0; e < rows * cols; ++e) {
      const int rl = e / cols, cl = e - rl * cols;
      const int row = wr * vw + rl, col = wc * vw + cl;
      if (!WX_CHK(row < gh && col < gw && excl + e < static_cast<long>(t) * gh * gw, 5003, row, col)) continue;
      window_index[s_tok_base + excl + e] = s_tok_base + (static_cast<long>(ti) * gh + row) * gw + col;
    }
  }
}

}  // namespace

WX_CHK_DEFINE_READER(index_check_read)

int rope_index(const long* ids, const int* mask, const int* img_grid, int n_img, const int* vid_grid, int n_vid,
               const float* sec_per_grid, int B, int S, int merge, long image_id, long video_id, long vstart_id,
               float tokens_per_second, long* pos, long* deltas, int* status, cudaStream_t s) {
  if (B == 0 || S == 0) return 0;
  const size_t smem = static_cast<size_t>(S) * 2 * sizeof(int);
  if (smem > 160 * 1024) return -1;
  static bool attr = false;
  if (!attr && smem > 32 * 1024) {
    cudaFuncSetAttribute(rope_index_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    attr = true;
  }
  rope_index_kernel<<<B, RI_THREADS, smem, s>>>(ids, mask, img_grid, n_img, vid_grid, n_vid, sec_per_grid, B, S, merge,
                                                image_id, video_id, vstart_id, tokens_per_second, pos, deltas, status);
  return static_cast<int>(cudaGetLastError());
}

int vit_rot_pos(const float* inv_freq, int F, const int* grid, int G, int merge, float* out, long N, cudaStream_t s) {
  const long total = N * F;
  if (total == 0) return 0;
  vit_rot_pos_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, s>>>(inv_freq, F, grid, G, merge, out, N);
  return static_cast<int>(cudaGetLastError());
}

int vit_window_index(const int* grid, int G, int vw, int merge, long* window_index, int* cu_seqlens, cudaStream_t s) {
  if (G == 0) return 0;
  vit_window_index_kernel<<<G, 256, 0, s>>>(grid, G, vw, merge, window_index, cu_seqlens);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace wx
