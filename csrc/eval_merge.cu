// Cross-rank merges of the sharded evaluation, by peer loads from the ranks' symmetric buffers (no library collective,
// no host round trip): sums of per-query partials (target scores, "greater" and "filtered" counts -> filtered ranks)
// and the merge of W x k top-k candidates per query.  Every rank runs the same merge over all queries; the buffers are
// tiny next to the scoring GEMM that produced them.  The reference ranks on one device with a dense sort
// (dicee/evaluation/evaluator.py:473-510) and takes torch.topk over all scores
// (dicee/knowledge_graph_embeddings.py:390-403).
#include "dice_b200.h"
#include "ptx_sm100.cuh"

namespace dice {

__global__ void peer_sum_f32_kernel(const float* const* table, int W, float* out, int n, const int* status) {
  if (status != nullptr && *status != 0) return;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s = 0.f;
  for (int k = 0; k < W; ++k) s += table[k][i];
  out[i] = s;
}

__global__ void merge_ranks_kernel(const int* const* greater, const int* const* filtered, int W, long long* ranks,
                                   int n, const int* status) {
  if (status != nullptr && *status != 0) return;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  long long r = 1;
  for (int k = 0; k < W; ++k) r += greater[k][i] - filtered[k][i];
  ranks[i] = r;
}

// One warp per query: the W * k candidates (k <= 32, W <= 8: at most 8 per lane) are held in registers and the best is
// extracted k times by a warp-wide arg-max (score descending, entity id ascending on ties).
__global__ void __launch_bounds__(256) merge_topk_kernel(const float* const* score, const long long* const* idx, int W,
                                                         int k, long long stride, float* out_s, long long* out_i,
                                                         int n, const int* status) {
  if (status != nullptr && *status != 0) return;
  const int lane = threadIdx.x & 31;
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (row >= n) return;
  const int total = W * k;
  float s[8];
  long long id[8];
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const int c = u * 32 + lane;
    s[u] = -INFINITY;
    id[u] = -1;
    if (c < total) {
      const int rk = c / k, j = c - rk * k;
      s[u] = score[rk][row * stride + j];
      id[u] = idx[rk][row * stride + j];
      if (id[u] < 0) s[u] = -INFINITY;   // empty slot of a rank that had fewer than k rows
    }
  }
  for (int t = 0; t < k; ++t) {
    float bs = -INFINITY;
    long long bi = -1;
    int bu = -1;
#pragma unroll
    for (int u = 0; u < 8; ++u)
      if (s[u] > bs || (s[u] == bs && bu >= 0 && id[u] >= 0 && id[u] < bi)) { bs = s[u]; bi = id[u]; bu = u; }
    float ws = bs;
    long long wi = bi;
    int wl = lane;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float os = __shfl_xor_sync(0xffffffffu, ws, o);
      const long long oi = __shfl_xor_sync(0xffffffffu, wi, o);
      const int ol = __shfl_xor_sync(0xffffffffu, wl, o);
      const bool better = os > ws || (os == ws && (oi >= 0 && (wi < 0 || oi < wi || (oi == wi && ol < wl))));
      if (better) { ws = os; wi = oi; wl = ol; }
    }
    if (lane == 0) {
      out_s[static_cast<long long>(row) * k + t] = ws;
      out_i[static_cast<long long>(row) * k + t] = wi;
    }
    if (lane == wl && bu >= 0) {   // the winning lane retires its candidate
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (u == bu) { s[u] = -INFINITY; id[u] = -1; }
    }
  }
}

}  // namespace dice

using namespace dice;

// out[i] = sum over the W buffers of table (device array of base pointers, peer memory allowed) of entry i.
extern "C" int dice_peer_sum_f32(const float* const* table, int W, float* out, int n, const int* status, void* stream) {
  if (n <= 0) return 0;
  peer_sum_f32_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(table, W, out, n, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// ranks[i] = 1 + sum_k greater[k][i] - sum_k filtered[k][i]
extern "C" int dice_merge_ranks(const int* const* greater, const int* const* filtered, int W, long long* ranks, int n,
                                const int* status, void* stream) {
  if (n <= 0) return 0;
  merge_ranks_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(greater, filtered, W, ranks, n,
                                                                                    status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Per query the best k of the W * k candidates found in score[rank][row * stride + j] / idx[...] (j < k); entries with
// a negative id are empty.  k <= 32 and W * k <= 256.
extern "C" int dice_merge_topk(const float* const* score, const long long* const* idx, int W, int k, long long stride,
                               float* out_s, long long* out_i, int n, const int* status, void* stream) {
  if (n <= 0) return 0;
  if (k < 1 || k > 32 || W * k > 256) return -6;
  const long long threads = static_cast<long long>(n) * 32;
  merge_topk_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      score, idx, W, k, stride, out_s, out_i, n, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
