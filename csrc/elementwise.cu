// Bandwidth-bound kernels around the fused scoring GEMM:
//   * lookup + query composition (+ broadcast of the bf16 query rows to every rank's buffer),
//   * sparse positive-label correction of loss / dQ / dE driven by the CSR of known tails,
//   * backward of the composition with scatter-add of row gradients to the owning shard,
//   * dense Adam / ADOPT / SGD sweeps that also refresh the bf16 shadow table and clear the gradient,
//   * small helpers (casts, prefix sums, loss finalisation).
// Entity rows are distributed cyclically: global row e lives on rank e % W at local row e / W.  All kernels take
// arrays of per-rank base pointers, so with W == 1 they act on one table and with W > 1 they read / write peer
// memory directly (plain ld/st/red over NVLink; no multicast loads).
#include "algebra.cuh"
#include "optim.cuh"
#include "ptx_sm100.cuh"
#include "launch_pdl.cuh"

namespace dice {

// Loads the K x VEC elements of row `row` that one thread owns (positions j0..j0+VEC-1 of every block).
template <int K, int VEC>
__device__ __forceinline__ void load_blocks(const float* __restrict__ row, int w, int j0, float (&v)[K][VEC]) {
#pragma unroll
  for (int a = 0; a < K; ++a)
#pragma unroll
    for (int u = 0; u < VEC; ++u) v[a][u] = row[a * w + j0 + u];
}

template <int K, int VEC>
__device__ __forceinline__ void normalize_rel(int mode, const float (&r)[K][VEC], float (&rh)[K][VEC],
                                              float (&nrm)[K][VEC]) {
#pragma unroll
  for (int a = 0; a < K; ++a)
#pragma unroll
    for (int u = 0; u < VEC; ++u) { rh[a][u] = r[a][u]; nrm[a][u] = 1.f; }
  if (mode == NORM_ACROSS_BLOCKS) {
#pragma unroll
    for (int u = 0; u < VEC; ++u) {
      float s = 0.f;
#pragma unroll
      for (int a = 0; a < K; ++a) s += r[a][u] * r[a][u];
      const float n = sqrtf(s);
#pragma unroll
      for (int a = 0; a < K; ++a) { rh[a][u] = r[a][u] / n; nrm[a][u] = n; }
    }
  } else if (mode == NORM_CONSECUTIVE4) {
#pragma unroll
    for (int a = 0; a < K; ++a) {
      float s = 0.f;
#pragma unroll
      for (int u = 0; u < VEC; ++u) s += r[a][u] * r[a][u];
      const float n = fmaxf(sqrtf(s), 1e-12f);
#pragma unroll
      for (int u = 0; u < VEC; ++u) { rh[a][u] = r[a][u] / n; nrm[a][u] = n; }
    }
  }
}

struct LookupParams {
  const long long* idx_h;        // [B] global entity ids
  const long long* idx_r;        // [B] relation ids
  const float* const* ent;       // [W] fp32 shard bases (peer pointers allowed)
  const float* rel;              // [R, D] replicated
  const float* coeff;            // Keci q-coefficient (single float) or null
  __nv_bfloat16* const* q_dst;   // [n_dst] destination query buffers (all ranks, or just this one)
  float* q_f32;                  // optional local fp32 copy [B, D]
  int n_dst;
  long long q_row_offset;        // first destination row of this rank's batch
  int B, D, W, norm_mode;
  int* status;
  long long num_entities;
  const long long* dp_src;       // optional: data-point ids of the batch, broadcast next to the queries
  long long* const* dp_dst;      // [n_dst] destinations (row offset q_row_offset)
  int additive;                  // translation models: q = h + r instead of the algebra product
};

template <int K, int VEC>
__global__ void lookup_compose_kernel(const LookupParams p) {
  const int w = p.D / K;
  const int per_row = w / VEC;
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (tid >= static_cast<long long>(p.B) * per_row) return;
  const int i = static_cast<int>(tid / per_row);
  const int j0 = static_cast<int>(tid % per_row) * VEC;
  const long long h = p.idx_h[i];
  const long long r_id = p.idx_r[i];
  if (h < 0 || h >= p.num_entities || r_id < 0) { atomicCAS(p.status, 0, ST_BAD_INDEX); return; }
  const float* hrow = p.ent[h % p.W] + (h / p.W) * p.D;
  const float* rrow = p.rel + r_id * p.D;
  if (j0 == 0 && p.dp_src != nullptr) {
    const long long d = p.dp_src[i];
    for (int k = 0; k < p.n_dst; ++k) p.dp_dst[k][p.q_row_offset + i] = d;
  }
  float hv[K][VEC], rv[K][VEC], rh[K][VEC], nrm[K][VEC];
  load_blocks<K, VEC>(hrow, w, j0, hv);
  load_blocks<K, VEC>(rrow, w, j0, rv);
  normalize_rel<K, VEC>(p.norm_mode, rv, rh, nrm);
  if (p.coeff != nullptr) {  // Keci Cl(0,1): the vector part of head and relation is scaled by the coefficient
    const float c = *p.coeff;
#pragma unroll
    for (int u = 0; u < VEC; ++u) { hv[K - 1][u] *= c; rh[K - 1][u] *= c; }
  }
#pragma unroll
  for (int k = 0; k < K; ++k) {
#pragma unroll
    for (int u = 0; u < VEC; ++u) {
      float q = 0.f;
#pragma unroll
      for (int a = 0; a < K; ++a) q = fmaf(Alg<K>::sgn(k, a) * hv[a][u], rh[Alg<K>::idx(k, a)][u], q);
      if (p.additive) q = hv[k][u] + rh[k][u];
      const long long col = k * w + j0 + u;
      const __nv_bfloat16 qb = __float2bfloat16_rn(q);
      for (int d = 0; d < p.n_dst; ++d) p.q_dst[d][(p.q_row_offset + i) * p.D + col] = qb;
      if (p.q_f32 != nullptr) p.q_f32[static_cast<long long>(i) * p.D + col] = q;
    }
  }
}

struct ComposeBwdParams {
  const long long* idx_h;
  const long long* idx_r;
  const float* const* ent;     // fp32 shards (forward values are recomputed from them)
  const float* rel;
  const float* coeff;
  const float* dq;             // [B, D] fp32 gradient w.r.t. the query vectors
  float* const* g_ent;         // [W] fp32 gradient shards (red.add; peer pointers allowed)
  float* g_rel;                // [R, D]
  float* g_coeff;              // single float or null
  int B, D, W, norm_mode;
  int additive;
  unsigned char* const* touched;  // optional [W] per-row flags of the gradient shards: set where a row gets a gradient
  // optional: dq of batch item i = sum over n_dq buffers (one per rank, peer pointers) of row dq_row_offset + i.
  // This is the consumer side of a reduce-scatter: every rank keeps its partial query gradients for the whole batch
  // locally and the owner of a batch slice sums the partials with coalesced peer loads while it applies the chain rule.
  const float* const* dq_table;
  int n_dq;
  long long dq_row_offset;
};

template <int K, int VEC>
__global__ void compose_backward_kernel(const ComposeBwdParams p) {
  const int w = p.D / K;
  const int per_row = w / VEC;
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  float dc = 0.f;
  if (tid < static_cast<long long>(p.B) * per_row) {
    const int i = static_cast<int>(tid / per_row);
    const int j0 = static_cast<int>(tid % per_row) * VEC;
    const long long h = p.idx_h[i];
    const long long r_id = p.idx_r[i];
    const float* hrow = p.ent[h % p.W] + (h / p.W) * p.D;
    const float* rrow = p.rel + r_id * p.D;
    float hv[K][VEC], rv[K][VEC], rh[K][VEC], nrm[K][VEC], dq[K][VEC], dh[K][VEC], drh[K][VEC];
    load_blocks<K, VEC>(hrow, w, j0, hv);
    load_blocks<K, VEC>(rrow, w, j0, rv);
    if (p.dq_table == nullptr) {
      load_blocks<K, VEC>(p.dq + static_cast<long long>(i) * p.D, w, j0, dq);
    } else {
#pragma unroll
      for (int a = 0; a < K; ++a)
#pragma unroll
        for (int u = 0; u < VEC; ++u) dq[a][u] = 0.f;
      for (int k = 0; k < p.n_dq; ++k) {
        float part[K][VEC];
        load_blocks<K, VEC>(p.dq_table[k] + (p.dq_row_offset + i) * p.D, w, j0, part);
#pragma unroll
        for (int a = 0; a < K; ++a)
#pragma unroll
          for (int u = 0; u < VEC; ++u) dq[a][u] += part[a][u];
      }
    }
    normalize_rel<K, VEC>(p.norm_mode, rv, rh, nrm);
    float c = 1.f;
    if (p.coeff != nullptr) {
      c = *p.coeff;
#pragma unroll
      for (int u = 0; u < VEC; ++u) { hv[K - 1][u] *= c; rh[K - 1][u] *= c; }
    }
#pragma unroll
    for (int a = 0; a < K; ++a)
#pragma unroll
      for (int u = 0; u < VEC; ++u) { dh[a][u] = 0.f; drh[a][u] = 0.f; }
#pragma unroll
    for (int k = 0; k < K; ++k)
#pragma unroll
      for (int a = 0; a < K; ++a)
#pragma unroll
        for (int u = 0; u < VEC; ++u) {
          const float g = Alg<K>::sgn(k, a) * dq[k][u];
          dh[a][u] = fmaf(g, rh[Alg<K>::idx(k, a)][u], dh[a][u]);
          drh[Alg<K>::idx(k, a)][u] = fmaf(g, hv[a][u], drh[Alg<K>::idx(k, a)][u]);
        }
    if (p.additive) {
#pragma unroll
      for (int a = 0; a < K; ++a)
#pragma unroll
        for (int u = 0; u < VEC; ++u) { dh[a][u] = dq[a][u]; drh[a][u] = dq[a][u]; }
    }
    if (p.coeff != nullptr) {
      // hv[K-1] = c * h_raw, rh[K-1] = c * r_raw  =>  d/dc collects both, raw grads pick up a factor c
#pragma unroll
      for (int u = 0; u < VEC; ++u) {
        const float h_raw = (c != 0.f) ? hv[K - 1][u] / c : hrow[(K - 1) * w + j0 + u];
        const float r_raw = (c != 0.f) ? rh[K - 1][u] / c : rrow[(K - 1) * w + j0 + u];
        dc += dh[K - 1][u] * h_raw + drh[K - 1][u] * r_raw;
        dh[K - 1][u] *= c;
        drh[K - 1][u] *= c;
      }
    }
    // back through the relation normalisation: dr = (drh - rh * <drh, rh>_group) / norm
    if (p.norm_mode == NORM_ACROSS_BLOCKS) {
#pragma unroll
      for (int u = 0; u < VEC; ++u) {
        float dot = 0.f;
#pragma unroll
        for (int a = 0; a < K; ++a) dot += drh[a][u] * rh[a][u];
#pragma unroll
        for (int a = 0; a < K; ++a) drh[a][u] = (drh[a][u] - rh[a][u] * dot) / nrm[a][u];
      }
    } else if (p.norm_mode == NORM_CONSECUTIVE4) {
#pragma unroll
      for (int a = 0; a < K; ++a) {
        float dot = 0.f;
#pragma unroll
        for (int u = 0; u < VEC; ++u) dot += drh[a][u] * rh[a][u];
#pragma unroll
        for (int u = 0; u < VEC; ++u) drh[a][u] = (drh[a][u] - rh[a][u] * dot) / nrm[a][u];
      }
    }
    float* ge = p.g_ent[h % p.W] + (h / p.W) * p.D;
    float* gr = p.g_rel + r_id * p.D;
    if (p.touched != nullptr && j0 == 0) p.touched[h % p.W][h / p.W] = 1;
#pragma unroll
    for (int a = 0; a < K; ++a)
#pragma unroll
      for (int u = 0; u < VEC; ++u) {
        atomicAdd(ge + a * w + j0 + u, dh[a][u]);
        atomicAdd(gr + a * w + j0 + u, drh[a][u]);
      }
  }
  if (p.g_coeff != nullptr) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dc += __shfl_xor_sync(0xffffffffu, dc, o);
    if ((threadIdx.x & 31) == 0 && dc != 0.f) atomicAdd(p.g_coeff, dc);
  }
}

// ------------------------------------------------------------------------------------ positives
// first[i] = number of positive labels of batch items 0..i-1; first[n] = total.  Two launches: the counts (two
// dependent random reads per item; spread over many SMs because one SM sustains too few outstanding misses for a
// large batch) and a one-block scan over the counts parked in first[].
__global__ void positive_count_kernel(const long long* __restrict__ dp_idx, const long long* __restrict__ offsets,
                                      int n, int* __restrict__ first, long long num_data_points, int* status) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long long d = dp_idx[i];
  if (num_data_points > 0 && (d < 0 || d >= num_data_points)) {   // reported; the item then has no positives
    if (status != nullptr) atomicCAS(status, 0, ST_BAD_INDEX);
    first[i] = 0;
    return;
  }
  first[i] = static_cast<int>(offsets[d + 1] - offsets[d]);
}

__global__ void positive_scan_kernel(int n, int* first) {
  // 32 warps; warp w owns the items [w * chunk, (w + 1) * chunk).  All reads and writes are coalesced 128-byte rows and
  // the reads of one group of eight rows are independent, so the single block is not bound by load latency.
  __shared__ int warp_tot[32];
  const unsigned full = 0xffffffffu;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int chunk = ((n + 1023) / 1024) * 32;
  const int lo = min(n, warp * chunk), hi = min(n, lo + chunk);
  int tot = 0;
#pragma unroll 8
  for (int i = lo + lane; i < hi; i += 32) tot += first[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(full, tot, o);
  if (lane == 0) warp_tot[warp] = tot;
  __syncthreads();
  if (warp == 0) {
    const int own = warp_tot[lane];
    int v = own;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(full, v, o);
      if (lane >= o) v += t;
    }
    warp_tot[lane] = v - own;   // exclusive prefix of the warp totals
  }
  __syncthreads();
  int carry = warp_tot[warp];
  for (int base = lo; base < hi; base += 256) {
    int c[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int i = base + k * 32 + lane;
      c[k] = i < hi ? first[i] : 0;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int i = base + k * 32 + lane;
      int v = c[k];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(full, v, o);
        if (lane >= o) v += t;
      }
      if (i < hi) first[i] = carry + v - c[k];
      carry += __shfl_sync(full, v, 31);
    }
  }
  if (warp == 31 && lane == 0) first[n] = carry;   // warps past the end have empty ranges: their carry is the total
}

struct PositiveParams {
  const long long* dp_idx;     // [n] data-point ids of the (gathered) batch
  const long long* offsets;    // CSR over data points
  const long long* values;     // global tail ids
  const int* first;            // [n + 1] prefix sums of positives per batch item
  const __nv_bfloat16* q;      // [n, D]
  const __nv_bfloat16* e;      // local entity shard [rows_local, D], bf16 shadow
  float* dq;                   // [n, D] fp32, red.add
  float* const* dq_table;      // optional: row i goes to dq_table[i / dq_block_rows] + (i % dq_block_rows) * D
  int dq_block_rows;
  float* de;                   // [rows_local, D] fp32, red.add
  double* loss;
  float weight;                // label(positive) - label(elsewhere)
  float scale;                 // 1 / (B * |E|)
  int n, W, rank;
};

__device__ __forceinline__ float* dq_row(const PositiveParams& p, int i, int D) {
  return p.dq_table != nullptr ? p.dq_table[i / p.dq_block_rows] + static_cast<long long>(i % p.dq_block_rows) * D
                               : p.dq + static_cast<long long>(i) * D;
}

template <int D, int CHUNK>
__global__ void positive_correction_kernel(const PositiveParams p) {
  constexpr int PER = D / 32;  // dims per lane
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const long long warp_global = blockIdx.x * static_cast<long long>(warps_per_block) + (threadIdx.x >> 5);
  const long long num_warps = static_cast<long long>(gridDim.x) * warps_per_block;
  const int total = p.first[p.n];
  float loss_local = 0.f;
  for (long long c0 = warp_global * CHUNK; c0 < total; c0 += num_warps * CHUNK) {
    const int pend = static_cast<int>(min(static_cast<long long>(total), c0 + CHUNK));
    // batch item owning positive c0: last i with first[i] <= c0
    int lo = 0, hi = p.n;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (p.first[mid] <= c0) lo = mid; else hi = mid;
    }
    int i = lo;
    float qv[PER], acc[PER];
    int loaded = -1;
#pragma unroll
    for (int u = 0; u < PER; ++u) acc[u] = 0.f;
    for (int pp = static_cast<int>(c0); pp < pend; ++pp) {
      while (p.first[i + 1] <= pp) {
        if (loaded == i) {
#pragma unroll
          for (int u = 0; u < PER; ++u) { atomicAdd(dq_row(p, i, D) + lane * PER + u, acc[u]); acc[u] = 0.f; }
        }
        ++i;
      }
      const long long d = p.dp_idx[i];
      const long long j = p.values[p.offsets[d] + (pp - p.first[i])];
      if (j % p.W != p.rank) continue;
      if (loaded != i) {
        const __nv_bfloat16* qrow = p.q + static_cast<long long>(i) * D + lane * PER;
#pragma unroll
        for (int u = 0; u < PER; ++u) qv[u] = __bfloat162float(qrow[u]);
        loaded = i;
      }
      const long long jl = j / p.W;
      const __nv_bfloat16* erow = p.e + jl * D + lane * PER;
      float ev[PER];
      float dot = 0.f;
#pragma unroll
      for (int u = 0; u < PER; ++u) { ev[u] = __bfloat162float(erow[u]); dot = fmaf(qv[u], ev[u], dot); }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      loss_local -= p.weight * dot;
      const float g = -p.weight * p.scale;
      float* derow = p.de + jl * D + lane * PER;
#pragma unroll
      for (int u = 0; u < PER; ++u) { atomicAdd(derow + u, g * qv[u]); acc[u] = fmaf(g, ev[u], acc[u]); }
    }
    if (loaded == i) {
#pragma unroll
      for (int u = 0; u < PER; ++u) atomicAdd(dq_row(p, i, D) + lane * PER + u, acc[u]);
    }
  }
  if (lane == 0 && loss_local != 0.f) atomicAdd(p.loss, static_cast<double>(loss_local));
}

// Label bit masks for the fused scoring kernel.  One warp per batch item walks its slice of the CSR and sets
//   mask_q[i][tail_local]   (rows = queries,  bit = local entity)   and
//   mask_e[tail_local][i]   (rows = entities, bit = query),
// keeping only tails owned by this rank.  Both masks are cleared by the caller before every batch.
__global__ void build_label_masks_kernel(const long long* __restrict__ dp_idx, const long long* __restrict__ offsets,
                                         const long long* __restrict__ values, int n, int W, int rank,
                                         unsigned int* __restrict__ mask_q, int stride_q,
                                         unsigned int* __restrict__ mask_e, int stride_e) {
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  if (warp >= n) return;
  const int i = static_cast<int>(warp);
  const long long d = dp_idx[i];
  const long long beg = offsets[d], end = offsets[d + 1];
  for (long long q = beg + lane; q < end; q += 32) {
    const long long j = values[q];
    if (j % W != rank) continue;
    const long long jl = j / W;
    atomicOr(mask_q + static_cast<long long>(i) * stride_q + (jl >> 5), 1u << (jl & 31));
    atomicOr(mask_e + jl * stride_e + (i >> 5), 1u << (i & 31));
  }
}

// Same result as build_label_masks_kernel, one thread per positive label: `first` holds the prefix sums of the
// positives per data point (positive_scan_kernel), a binary search finds the data point of a positive.  A few data
// points of a Zipf-shaped graph have thousands of known tails; with one warp per data point those few warps set the
// kernel's duration.
__global__ void build_label_masks_flat_kernel(const long long* __restrict__ dp_idx,
                                              const long long* __restrict__ offsets,
                                              const long long* __restrict__ values, const int* __restrict__ first,
                                              int n, int W, int rank, unsigned int* __restrict__ mask_q, int stride_q,
                                              unsigned int* __restrict__ mask_e, int stride_e,
                                              long long num_local_rows, int* status) {
  const int total = first[n];
  const int stride = gridDim.x * blockDim.x;
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    int lo = 0, hi = n - 1;  // largest i with first[i] <= t
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (first[mid] <= t) lo = mid; else hi = mid - 1;
    }
    const int i = lo;
    const long long j = values[offsets[dp_idx[i]] + (t - first[i])];
    if (j % W != rank) continue;
    const long long jl = j / W;
    if (num_local_rows > 0 && (j < 0 || jl >= num_local_rows)) {   // a CSR value outside the local shard
      if (status != nullptr) atomicCAS(status, 0, ST_BAD_INDEX);
      continue;
    }
    atomicOr(mask_q + static_cast<long long>(i) * stride_q + (jl >> 5), 1u << (jl & 31));
    atomicOr(mask_e + jl * stride_e + (i >> 5), 1u << (i & 31));
  }
}

// Same result in ONE launch and without a global prefix sum: a block takes MASK_ITEMS consecutive batch items, scans
// their positive counts in shared memory and then deals the block's positives to its threads one by one (binary search
// in the shared prefix array).  Work is balanced inside a block; an item with thousands of known tails makes its block
// loop a few more times, which costs microseconds, while the three dependent launches of the scan-based variant cost
// about 20 us on the critical path of a training step.
constexpr int MASK_ITEMS = 64;
__global__ void __launch_bounds__(256) build_label_masks_block_kernel(
    const long long* __restrict__ dp_idx, const long long* __restrict__ offsets, const long long* __restrict__ values,
    int n, int W, int rank, unsigned int* __restrict__ mask_q, int stride_q, unsigned int* __restrict__ mask_e,
    int stride_e, long long num_data_points, long long num_local_rows, int* status) {
  __shared__ int pre[MASK_ITEMS + 1];
  __shared__ long long beg[MASK_ITEMS];
  const int i0 = blockIdx.x * MASK_ITEMS;
  const int items = min(MASK_ITEMS, n - i0);
  if (threadIdx.x < MASK_ITEMS) {
    int c = 0;
    long long b = 0;
    if (threadIdx.x < items) {
      const long long d = dp_idx[i0 + threadIdx.x];
      if (num_data_points > 0 && (d < 0 || d >= num_data_points)) {
        if (status != nullptr) atomicCAS(status, 0, ST_BAD_INDEX);
      } else {
        b = offsets[d];
        c = static_cast<int>(offsets[d + 1] - b);
      }
    }
    beg[threadIdx.x] = b;
    // inclusive scan over the 64 counts: two warps, then the second adds the first warp's total
    int v = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, v, o);
      if ((threadIdx.x & 31) >= o) v += t;
    }
    pre[threadIdx.x + 1] = v;
  }
  __syncthreads();
  if (threadIdx.x >= 32 && threadIdx.x < MASK_ITEMS) pre[threadIdx.x + 1] += pre[32];
  if (threadIdx.x == 0) pre[0] = 0;
  __syncthreads();
  const int total = pre[MASK_ITEMS];
  for (int t = threadIdx.x; t < total; t += blockDim.x) {
    int lo = 0, hi = MASK_ITEMS - 1;   // largest k with pre[k] <= t
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (pre[mid] <= t) lo = mid; else hi = mid - 1;
    }
    const int i = i0 + lo;
    const long long j = values[beg[lo] + (t - pre[lo])];
    if (j % W != rank) continue;
    const long long jl = j / W;
    if (num_local_rows > 0 && (j < 0 || jl >= num_local_rows)) {
      if (status != nullptr) atomicCAS(status, 0, ST_BAD_INDEX);
      continue;
    }
    atomicOr(mask_q + static_cast<long long>(i) * stride_q + (jl >> 5), 1u << (jl & 31));
    atomicOr(mask_e + jl * stride_e + (i >> 5), 1u << (i & 31));
  }
}

// ------------------------------------------------------------------------------------ optimisers
struct OptParams {
  float* param;
  float* grad;               // cleared after use
  float* m;
  float* v;
  __nv_bfloat16* shadow;     // optional bf16 copy refreshed in the same pass
  const long long* step;     // device-side step counter (number of completed steps)
  long long n;
  float lr, beta1, beta2, eps, weight_decay;
  int kind;                  // 0 Adam, 1 AdamW, 2 SGD, 3 ADOPT
  const float* const* grad_table;  // optional: gradient = sum over n_grad buffers (one per rank, peer pointers):
  int n_grad;                      // the all-reduce of replicated parameters folded into their update
  const float* grad_mc;            // optional: multicast address of the gradient buffer; the sum over all bound GPUs
                                   // is then formed inside the switch by multimem.ld_reduce (replaces grad_table)
  const int* status;               // optional: the sweep is skipped when this word already holds an error
};

__device__ __forceinline__ float4 opt_multimem_sum4(const float* mc_addr) {
  float4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w)
               : "l"(mc_addr)
               : "memory");
  return r;
}
__device__ __forceinline__ float opt_multimem_sum1(const float* mc_addr) {
  float r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.f32 %0, [%1];" : "=f"(r) : "l"(mc_addr) : "memory");
  return r;
}

__global__ void __launch_bounds__(256) optimizer_kernel(const OptParams p) {
  if (p.status != nullptr && *p.status != 0) return;
  const long long t = *p.step + 1;
  float inv_bc1 = 1.f, inv_sqrt_bc2 = 1.f;
  if (p.kind <= 1) {
    inv_bc1 = 1.f / (1.f - exp2f(static_cast<float>(t) * log2f(p.beta1)));
    inv_sqrt_bc2 = rsqrtf(1.f - exp2f(static_cast<float>(t) * log2f(p.beta2)));
  }
  const float clip = sqrtf(sqrtf(static_cast<float>(t - 1)));  // ADOPT: clip bound step^(1/4)
  const bool first_step = (t == 1);
  float* __restrict__ param = p.param;
  float* __restrict__ grad = p.grad;
  float* __restrict__ pm = p.m;
  float* __restrict__ pv = p.v;
  __nv_bfloat16* __restrict__ shadow = p.shadow;
  const long long n4 = p.n >> 2;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const bool aligned = ((reinterpret_cast<uintptr_t>(param) | reinterpret_cast<uintptr_t>(grad) |
                         reinterpret_cast<uintptr_t>(pm) | reinterpret_cast<uintptr_t>(pv)) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(shadow) & 7) == 0;
  bool table_aligned = true;  // gradient buffers of the ranks (symmetric-heap regions) are 16-byte aligned as a rule
  const bool remote = p.grad_table != nullptr || p.grad_mc != nullptr;   // gradient summed over ranks; owners clear later
  if (p.grad_mc != nullptr) table_aligned = (reinterpret_cast<uintptr_t>(p.grad_mc) & 15) == 0;
  else if (p.grad_table != nullptr)
    for (int k = 0; k < p.n_grad; ++k) table_aligned &= (reinterpret_cast<uintptr_t>(p.grad_table[k]) & 15) == 0;
  long long done = 0;
  if (aligned && table_aligned) {
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4; i += stride) {
      float4 w = reinterpret_cast<float4*>(param)[i];
      float4 g;
      if (p.grad_mc != nullptr) {     // sum of all ranks' buffers formed inside the switch
        g = opt_multimem_sum4(p.grad_mc + (i << 2));
      } else if (p.grad_table != nullptr) {  // sum of all ranks' buffers (peer loads): the all-reduce happens here
        g = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k = 0; k < p.n_grad; ++k) {
          const float4 t = reinterpret_cast<const float4*>(p.grad_table[k])[i];
          g.x += t.x; g.y += t.y; g.z += t.z; g.w += t.w;
        }
      } else {
        g = reinterpret_cast<float4*>(grad)[i];
      }
      float4 m = make_float4(0.f, 0.f, 0.f, 0.f), v = m;
      if (p.kind != 2) {
        m = reinterpret_cast<float4*>(pm)[i];
        v = reinterpret_cast<float4*>(pv)[i];
      }
      w.x = opt_update(p.kind, w.x, g.x, m.x, v.x, p.lr, p.beta1, p.beta2, p.eps, p.weight_decay, inv_bc1, inv_sqrt_bc2, clip, first_step);
      w.y = opt_update(p.kind, w.y, g.y, m.y, v.y, p.lr, p.beta1, p.beta2, p.eps, p.weight_decay, inv_bc1, inv_sqrt_bc2, clip, first_step);
      w.z = opt_update(p.kind, w.z, g.z, m.z, v.z, p.lr, p.beta1, p.beta2, p.eps, p.weight_decay, inv_bc1, inv_sqrt_bc2, clip, first_step);
      w.w = opt_update(p.kind, w.w, g.w, m.w, v.w, p.lr, p.beta1, p.beta2, p.eps, p.weight_decay, inv_bc1, inv_sqrt_bc2, clip, first_step);
      reinterpret_cast<float4*>(param)[i] = w;
      if (!remote) reinterpret_cast<float4*>(grad)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (p.kind != 2) {
        reinterpret_cast<float4*>(pm)[i] = m;
        reinterpret_cast<float4*>(pv)[i] = v;
      }
      if (shadow != nullptr) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(w.x, w.y), hi = __floats2bfloat162_rn(w.z, w.w);
        uint2 pk;
        pk.x = *reinterpret_cast<uint32_t*>(&lo);
        pk.y = *reinterpret_cast<uint32_t*>(&hi);
        reinterpret_cast<uint2*>(shadow)[i] = pk;
      }
    }
    done = n4 << 2;
  }
  for (long long i = done + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < p.n; i += stride) {
    float w = param[i];
    float g;
    if (p.grad_mc != nullptr) {
      g = opt_multimem_sum1(p.grad_mc + i);
    } else if (p.grad_table != nullptr) {
      g = 0.f;
      for (int k = 0; k < p.n_grad; ++k) g += p.grad_table[k][i];  // owners clear their buffer after the next barrier
    } else {
      g = grad[i];
      grad[i] = 0.f;
    }
    float m = 0.f, v = 0.f;
    if (p.kind != 2) { m = pm[i]; v = pv[i]; }
    w = opt_update(p.kind, w, g, m, v, p.lr, p.beta1, p.beta2, p.eps, p.weight_decay, inv_bc1, inv_sqrt_bc2, clip, first_step);
    param[i] = w;
    if (p.kind != 2) { pm[i] = m; pv[i] = v; }
    if (shadow != nullptr) shadow[i] = __float2bfloat16_rn(w);
  }
}

// ------------------------------------------------------------------------------------ end of a step in one launch
// Up to three parameter segments (entity shard, relation table, coefficient) are updated by one grid, and the block
// that finishes last closes the step: loss = accumulator / count, accumulator = 0, step += 1.  Every block reads the
// step counter when it starts, and the last block to finish is by construction behind all of those reads, so the
// increment cannot race with them.
struct StepTailParams {
  OptParams seg[3];
  int n_seg;
  double* acc;
  float* loss_out;
  double inv_count;
  long long* step_rw;
  const double* const* acc_table;
  int n_acc;
  unsigned int* done;          // zero-initialised counter, reset by the closing block
  const int* status;
};

__device__ __forceinline__ void optimizer_segment(const OptParams& p, long long t) {
  float inv_bc1 = 1.f, inv_sqrt_bc2 = 1.f;
  if (p.kind <= 1) {
    inv_bc1 = 1.f / (1.f - exp2f(static_cast<float>(t) * log2f(p.beta1)));
    inv_sqrt_bc2 = rsqrtf(1.f - exp2f(static_cast<float>(t) * log2f(p.beta2)));
  }
  const float clip = sqrtf(sqrtf(static_cast<float>(t - 1)));
  const bool first_step = (t == 1);
  const bool remote = p.grad_table != nullptr || p.grad_mc != nullptr;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  bool vec = ((reinterpret_cast<uintptr_t>(p.param) | reinterpret_cast<uintptr_t>(p.grad) |
               reinterpret_cast<uintptr_t>(p.m) | reinterpret_cast<uintptr_t>(p.v)) & 15) == 0 &&
             (reinterpret_cast<uintptr_t>(p.shadow) & 7) == 0;
  if (p.grad_mc != nullptr) vec &= (reinterpret_cast<uintptr_t>(p.grad_mc) & 15) == 0;
  else if (p.grad_table != nullptr)
    for (int k = 0; k < p.n_grad; ++k) vec &= (reinterpret_cast<uintptr_t>(p.grad_table[k]) & 15) == 0;
  long long done = 0;
  if (vec) {
    const long long n4 = p.n >> 2;
    for (long long i = tid; i < n4; i += stride) {
      float4 w = reinterpret_cast<float4*>(p.param)[i];
      float4 g;
      if (p.grad_mc != nullptr) {
        g = opt_multimem_sum4(p.grad_mc + (i << 2));
      } else if (p.grad_table != nullptr) {
        g = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k = 0; k < p.n_grad; ++k) {
          const float4 x = reinterpret_cast<const float4*>(p.grad_table[k])[i];
          g.x += x.x; g.y += x.y; g.z += x.z; g.w += x.w;
        }
      } else {
        g = reinterpret_cast<float4*>(p.grad)[i];
      }
      float4 m = make_float4(0.f, 0.f, 0.f, 0.f), v = m;
      if (p.kind != 2) {
        m = reinterpret_cast<float4*>(p.m)[i];
        v = reinterpret_cast<float4*>(p.v)[i];
      }
      w.x = opt_update(p.kind, w.x, g.x, m.x, v.x, p.lr, p.beta1, p.beta2, p.eps, p.weight_decay, inv_bc1, inv_sqrt_bc2, clip, first_step);
      w.y = opt_update(p.kind, w.y, g.y, m.y, v.y, p.lr, p.beta1, p.beta2, p.eps, p.weight_decay, inv_bc1, inv_sqrt_bc2, clip, first_step);
      w.z = opt_update(p.kind, w.z, g.z, m.z, v.z, p.lr, p.beta1, p.beta2, p.eps, p.weight_decay, inv_bc1, inv_sqrt_bc2, clip, first_step);
      w.w = opt_update(p.kind, w.w, g.w, m.w, v.w, p.lr, p.beta1, p.beta2, p.eps, p.weight_decay, inv_bc1, inv_sqrt_bc2, clip, first_step);
      reinterpret_cast<float4*>(p.param)[i] = w;
      if (!remote) reinterpret_cast<float4*>(p.grad)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (p.kind != 2) {
        reinterpret_cast<float4*>(p.m)[i] = m;
        reinterpret_cast<float4*>(p.v)[i] = v;
      }
      if (p.shadow != nullptr) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(w.x, w.y), hi = __floats2bfloat162_rn(w.z, w.w);
        uint2 pk;
        pk.x = *reinterpret_cast<uint32_t*>(&lo);
        pk.y = *reinterpret_cast<uint32_t*>(&hi);
        reinterpret_cast<uint2*>(p.shadow)[i] = pk;
      }
    }
    done = n4 << 2;
  }
  for (long long i = done + tid; i < p.n; i += stride) {
    float w = p.param[i];
    float g;
    if (p.grad_mc != nullptr) {
      g = opt_multimem_sum1(p.grad_mc + i);
    } else if (p.grad_table != nullptr) {
      g = 0.f;
      for (int k = 0; k < p.n_grad; ++k) g += p.grad_table[k][i];
    } else {
      g = p.grad[i];
      p.grad[i] = 0.f;
    }
    float m = 0.f, v = 0.f;
    if (p.kind != 2) { m = p.m[i]; v = p.v[i]; }
    w = opt_update(p.kind, w, g, m, v, p.lr, p.beta1, p.beta2, p.eps, p.weight_decay, inv_bc1, inv_sqrt_bc2, clip, first_step);
    p.param[i] = w;
    if (p.kind != 2) { p.m[i] = m; p.v[i] = v; }
    if (p.shadow != nullptr) p.shadow[i] = __float2bfloat16_rn(w);
  }
}

__global__ void __launch_bounds__(256) step_tail_kernel(const StepTailParams p) {
  griddep_wait();
  if (p.status != nullptr && *p.status != 0) return;
  const long long t = *p.step_rw + 1;
  for (int s = 0; s < p.n_seg; ++s) optimizer_segment(p.seg[s], t);
  if (p.done == nullptr) return;
  __shared__ bool last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last = atomicAdd(p.done, 1u) == gridDim.x - 1;
  __syncthreads();
  if (last && threadIdx.x == 0) {
    __threadfence();
    if (p.acc_table != nullptr) {
      double sum = 0.0;
      for (int k = 0; k < p.n_acc; ++k) sum += *p.acc_table[k];
      *p.loss_out = static_cast<float>(sum * p.inv_count);
    } else {
      *p.loss_out = static_cast<float>(*p.acc * p.inv_count);
      *p.acc = 0.0;
    }
    *p.step_rw = t;
    *p.done = 0u;
  }
}

__global__ void cast_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[i] = __float2bfloat16_rn(src[i]);
}

// loss_out = acc * inv_count; acc = 0; step += 1   (one thread)
// With acc_table the loss is the sum of every rank's accumulator (peer reads); each owner clears its own later.
__global__ void finish_step_kernel(double* acc, float* loss_out, double inv_count, long long* step,
                                   const double* const* acc_table, int n_acc, const int* status) {
  if (status != nullptr && *status != 0) return;
  if (acc_table != nullptr) {
    double s = 0.0;
    for (int k = 0; k < n_acc; ++k) s += *acc_table[k];
    *loss_out = static_cast<float>(s * inv_count);
  } else {
    *loss_out = static_cast<float>(*acc * inv_count);
    *acc = 0.0;
  }
  if (step != nullptr) *step += 1;
}

// Barrier across W ranks (one process per GPU) on per-rank signal arrays in peer-accessible memory.
// Rank r adds 1 to slot r of every peer's array, then waits until every slot of its own array reaches the
// number of barriers passed so far.  The wait is bounded; on a time-out the status word is set and the kernel
// returns, so the host sees an error instead of a hang.  Once the status word holds an error the barrier neither
// signals nor waits, and the kernels behind it that touch peer memory return at once.
__global__ void p2p_barrier_kernel(unsigned int* const* sig_table, int rank, int W, unsigned int* count, int* status,
                                   unsigned int spin_limit) {
  __shared__ unsigned int target;
  __shared__ int failed;
  if (threadIdx.x == 0) {
    target = *count + 1;
    *count = target;
    failed = *status;   // after a failure nothing is signalled any more: the peers' waits run out as well
  }
  __syncthreads();
  const int peer = threadIdx.x;
  if (peer < W && failed == 0) {
    __threadfence_system();
    asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(sig_table[peer] + rank) : "memory");
    const unsigned int* mine = sig_table[rank] + peer;
    unsigned int v = 0, it = 0;
    for (; it < spin_limit; ++it) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if (static_cast<int>(v - target) >= 0) break;
      if (it > 64) __nanosleep(100);
    }
    if (it >= spin_limit) atomicCAS(status, 0, ST_TIMEOUT_PEER);
    __threadfence_system();
  }
}

template <int K, int VEC>
static int launch_lookup(const LookupParams& p, cudaStream_t s) {
  const long long n = static_cast<long long>(p.B) * (p.D / K / VEC);
  lookup_compose_kernel<K, VEC><<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
template <int K, int VEC>
static int launch_bwd(const ComposeBwdParams& p, cudaStream_t s) {
  const long long n = static_cast<long long>(p.B) * (p.D / K / VEC);
  compose_backward_kernel<K, VEC><<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace dice

using namespace dice;

// model: 0 DistMult, 1 ComplEx, 2 QMult (relation quaternion-normalised over consecutive 4-tuples when
// normalize != 0), 3 OMult (relation normalised across its 8 blocks when normalize != 0), 4 Keci Cl(0,1) with
// coefficient `coeff`, 5 translation (q = h + r).  ent / q_dst are *device* arrays of W / n_dst base pointers.
extern "C" int dice_lookup_compose(int model, int normalize, const long long* idx_h, const long long* idx_r,
                                   const float* const* ent, int W, long long num_entities, const float* rel,
                                   const float* coeff, __nv_bfloat16* const* q_dst, int n_dst,
                                   long long q_row_offset, float* q_f32, int B, int D, int* status,
                                   const long long* dp_src, long long* const* dp_dst, void* stream) {
  if (B <= 0) return 0;
  LookupParams p{idx_h, idx_r, ent, rel, nullptr, q_dst, q_f32, n_dst, q_row_offset, B, D, W, NORM_NONE, status,
                 num_entities, dp_src, dp_dst};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (model) {
    case 0: return launch_lookup<1, 1>(p, s);
    case 1: if (D % 2) return -6; return launch_lookup<2, 1>(p, s);
    case 2: if (D % 16) return -6; p.norm_mode = normalize ? NORM_CONSECUTIVE4 : NORM_NONE; return launch_lookup<4, 4>(p, s);
    case 3: if (D % 8) return -6; p.norm_mode = normalize ? NORM_ACROSS_BLOCKS : NORM_NONE; return launch_lookup<8, 1>(p, s);
    case 4: if (D % 2) return -6; p.coeff = coeff; return launch_lookup<2, 1>(p, s);
    case 5: p.additive = 1; return launch_lookup<1, 1>(p, s);
    default: return -6;
  }
}

extern "C" int dice_compose_backward(int model, int normalize, const long long* idx_h, const long long* idx_r,
                                     const float* const* ent, int W, const float* rel, const float* coeff,
                                     const float* dq, float* const* g_ent, float* g_rel, float* g_coeff, int B, int D,
                                     unsigned char* const* touched, const float* const* dq_table, int n_dq,
                                     long long dq_row_offset, void* stream) {
  if (B <= 0) return 0;
  ComposeBwdParams p{idx_h, idx_r, ent, rel, nullptr, dq, g_ent, g_rel, nullptr, B, D, W, NORM_NONE, 0, touched,
                     dq_table, n_dq, dq_row_offset};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (model) {
    case 0: return launch_bwd<1, 1>(p, s);
    case 1: return launch_bwd<2, 1>(p, s);
    case 2: p.norm_mode = normalize ? NORM_CONSECUTIVE4 : NORM_NONE; return launch_bwd<4, 4>(p, s);
    case 3: p.norm_mode = normalize ? NORM_ACROSS_BLOCKS : NORM_NONE; return launch_bwd<8, 1>(p, s);
    case 4: p.coeff = coeff; p.g_coeff = g_coeff; return launch_bwd<2, 1>(p, s);
    case 5: p.additive = 1; return launch_bwd<1, 1>(p, s);
    default: return -6;
  }
}

extern "C" int dice_build_label_masks(const long long* dp_idx, const long long* offsets, const long long* values, int n,
                                      int W, int rank, unsigned int* mask_q, int stride_q, unsigned int* mask_e,
                                      int stride_e, void* stream) {
  if (n <= 0) return 0;
  const int threads = 256;
  const long long blocks = (static_cast<long long>(n) * 32 + threads - 1) / threads;
  build_label_masks_kernel<<<static_cast<unsigned>(blocks), threads, 0, static_cast<cudaStream_t>(stream)>>>(
      dp_idx, offsets, values, n, W, rank, mask_q, stride_q, mask_e, stride_e);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// first: int[n + 1] scratch for the prefix sums of positives per data point.
// first == null selects the one-launch variant (block-local prefix sums); otherwise first is int[n + 1] scratch for the
// count / scan / spread variant.  num_data_points / num_local_rows > 0 (with status) switch on range checks of the data-point ids and of the CSR
// values; offending entries are reported through *status and skipped.
extern "C" int dice_build_label_masks_flat(const long long* dp_idx, const long long* offsets, const long long* values,
                                           int* first, int n, int W, int rank, unsigned int* mask_q, int stride_q,
                                           unsigned int* mask_e, int stride_e, long long num_data_points,
                                           long long num_local_rows, int* status, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (first == nullptr) {   // one launch, block-local prefix sums
    build_label_masks_block_kernel<<<(n + MASK_ITEMS - 1) / MASK_ITEMS, 256, 0, s>>>(
        dp_idx, offsets, values, n, W, rank, mask_q, stride_q, mask_e, stride_e, num_data_points, num_local_rows,
        status);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
  }
  positive_count_kernel<<<(n + 255) / 256, 256, 0, s>>>(dp_idx, offsets, n, first, num_data_points, status);
  positive_scan_kernel<<<1, 1024, 0, s>>>(n, first);
  build_label_masks_flat_kernel<<<148 * 4, 256, 0, s>>>(dp_idx, offsets, values, first, n, W, rank, mask_q, stride_q,
                                                        mask_e, stride_e, num_local_rows, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int dice_positive_scan(const long long* dp_idx, const long long* offsets, int n, int* first, void* stream) {
  positive_count_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(dp_idx, offsets, n, first, 0,
                                                                                          nullptr);
  positive_scan_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(n, first);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int dice_positive_correction(const long long* dp_idx, const long long* offsets, const long long* values,
                                        const int* first, const void* q, const void* e, float* dq, float* de,
                                        double* loss, float weight, float scale, int n, int D, int W, int rank,
                                        float* const* dq_table, int dq_block_rows, void* stream) {
  if (n <= 0) return 0;
  PositiveParams p{dp_idx, offsets, values, first, static_cast<const __nv_bfloat16*>(q),
                   static_cast<const __nv_bfloat16*>(e), dq, dq_table, dq_block_rows > 0 ? dq_block_rows : 1, de, loss,
                   weight, scale, n, W, rank};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int blocks = 148 * 4, threads = 256;
  switch (D) {
    case 256: positive_correction_kernel<256, 8><<<blocks, threads, 0, s>>>(p); break;
    case 128: positive_correction_kernel<128, 8><<<blocks, threads, 0, s>>>(p); break;
    case 64: positive_correction_kernel<64, 8><<<blocks, threads, 0, s>>>(p); break;
    case 32: positive_correction_kernel<32, 8><<<blocks, threads, 0, s>>>(p); break;
    default: return -6;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int dice_optimizer_step(int kind, float* param, float* grad, float* m, float* v, void* shadow,
                                   const long long* step, long long n, float lr, float beta1, float beta2, float eps,
                                   float weight_decay, const float* const* grad_table, int n_grad,
                                   const float* grad_mc, const int* status, void* stream) {
  if (n <= 0) return 0;
  OptParams p{param, grad, m, v, static_cast<__nv_bfloat16*>(shadow), step, n, lr, beta1, beta2, eps, weight_decay, kind,
              grad_table, n_grad, grad_mc, status};
  const int threads = 256;
  long long blocks = (n + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  optimizer_kernel<<<static_cast<unsigned>(blocks), threads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// One launch for the end of a training step: optimiser sweeps over n_seg <= 3 parameter segments and, when `done`
// (a zero-initialised device counter) is given, the closing of the step by the last block.  Per segment s the arrays
// hold: param, grad, m, v, shadow (bf16 or null), n, grad_table (or null), grad_mc (or null); the optimiser kind and
// hyper-parameters are shared.  n_grad: number of buffers behind every non-null grad_table.
extern "C" int dice_step_tail(int kind, int n_seg, float* const* param, float* const* grad, float* const* m,
                              float* const* v, void* const* shadow, const long long* n,
                              const float* const* const* grad_table, const float* const* grad_mc, int n_grad,
                              long long* step, float lr, float beta1, float beta2, float eps, float weight_decay,
                              double* acc, float* loss_out, double inv_count, const double* const* acc_table, int n_acc,
                              unsigned int* done, const int* status, void* stream) {
  if (n_seg < 1 || n_seg > 3) return -6;
  StepTailParams p{};
  long long total = 0;
  for (int s = 0; s < n_seg; ++s) {
    p.seg[s] = OptParams{param[s], grad[s], m[s], v[s], static_cast<__nv_bfloat16*>(shadow[s]), step, n[s], lr, beta1,
                         beta2, eps, weight_decay, kind, grad_table ? grad_table[s] : nullptr, n_grad,
                         grad_mc ? grad_mc[s] : nullptr, status};
    total += n[s];
  }
  p.n_seg = n_seg;
  p.acc = acc; p.loss_out = loss_out; p.inv_count = inv_count; p.step_rw = step; p.acc_table = acc_table;
  p.n_acc = n_acc; p.done = done; p.status = status;
  const int threads = 256;
  long long blocks = (total / 4 + threads - 1) / threads;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (launch_pdl(step_tail_kernel, dim3(static_cast<unsigned>(blocks)), dim3(threads), 0,
                 static_cast<cudaStream_t>(stream), p) != cudaSuccess)
    return -4;
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int dice_cast_bf16(const float* src, void* dst, long long n, void* stream) {
  if (n <= 0) return 0;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  cast_bf16_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      src, static_cast<__nv_bfloat16*>(dst), n);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int dice_finish_step(double* acc, float* loss_out, double inv_count, long long* step,
                                const double* const* acc_table, int n_acc, const int* status, void* stream) {
  finish_step_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(acc, loss_out, inv_count, step, acc_table, n_acc,
                                                                      status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Writes the GPU's nanosecond timer into *slot: launched between the kernels of a (captured) step it gives per-phase
// device times without host events.
__global__ void timestamp_kernel(unsigned long long* slot) {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  *slot = t;
}
extern "C" int dice_timestamp(unsigned long long* slot, void* stream) {
  timestamp_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(slot);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// sig_table: device array of W pointers to each rank's unsigned[W] signal array; count: this rank's barrier counter.
extern "C" int dice_p2p_barrier(unsigned int* const* sig_table, int rank, int W, unsigned int* count, int* status,
                                unsigned int spin_limit, void* stream) {
  if (W <= 1) return 0;
  if (W > 64) return -6;
  p2p_barrier_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(sig_table, rank, W, count, status,
                                                                      spin_limit ? spin_limit : (1u << 24));
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// ------------------------------------------------------------------------------------ allocation-free entry point
// Sparse positive-label correction for callers that must not allocate device memory.
//
// dice_positive_scan + dice_positive_correction need an int[n + 1] prefix-sum buffer that the caller allocates.
// Some callers cannot do that: code running inside a CUDA-graph capture or a stream-ordered region where
// cudaMalloc is illegal or would synchronise the device, plug-ins living inside another framework's memory
// budget (a serving process that has handed all free memory to its own pool), and hosts written in languages
// whose binding layer has no allocator hooked up.  For them the prefix sums live in a fixed array inside the
// library image instead.
//
// * Capacity: n <= DICE_NOALLOC_MAX_BATCH batch items; larger n is rejected with -7 and a message on stderr.
// * The array (DICE_NOALLOC_MAX_BATCH + 1 ints, 256 KiB) is part of the loaded library: every GPU that loads
//   the library carries it until the process exits.
// * The first call on each device looks up the device address of the array (cudaGetSymbolAddress) with that
//   device current and caches it; make that first call outside any stream capture.
// * All calls share the one array and it keeps the previous call's contents.  Nothing in it has to start at zero
//   (the scan overwrites entries 0..n before the correction kernel reads them), but two calls whose kernels
//   overlap on the GPU (different streams, or different host threads on one device) race on it: serialise them.
// * Neither this function nor the kernels it launches call cudaMalloc, cudaFree or any allocating routine.
#include "dice_b200.h"

#include <stdio.h>

#include <mutex>

namespace dice {
static __device__ __align__(256) int g_noalloc_first[DICE_NOALLOC_MAX_BATCH + 1];
static int* g_noalloc_first_addr[64] = {nullptr};
static std::mutex g_noalloc_mutex;
}  // namespace dice

extern "C" int dice_positive_correction_noalloc(const long long* dp_idx, const long long* offsets,
                                                const long long* values, const void* q, const void* e, float* dq,
                                                float* de, double* loss, float weight, float scale, int n, int D,
                                                int W, int rank, void* stream) {
  if (n <= 0) return 0;
  if (n > DICE_NOALLOC_MAX_BATCH) {
    fprintf(stderr, "dice_positive_correction_noalloc: n = %d exceeds the built-in scratch capacity of %d batch items\n",
            n, DICE_NOALLOC_MAX_BATCH);
    return -7;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -8;
  int* first = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (g_noalloc_first_addr[dev] == nullptr) {
      // In host code the array's name is only a handle; the kernels need its address on the current device.
      void* addr = nullptr;
      const cudaError_t rc = cudaGetSymbolAddress(&addr, g_noalloc_first);
      if (rc != cudaSuccess || addr == nullptr) {
        fprintf(stderr, "dice_positive_correction_noalloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(rc));
        return -9;
      }
      g_noalloc_first_addr[dev] = static_cast<int*>(addr);
    }
    first = g_noalloc_first_addr[dev];
  }
  int rc = dice_positive_scan(dp_idx, offsets, n, first, stream);
  if (rc != 0) return rc;
  return dice_positive_correction(dp_idx, offsets, values, first, q, e, dq, de, loss, weight, scale, n, D, W, rank,
                                  nullptr, 0, stream);
}
