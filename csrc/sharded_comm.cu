// Vectorised lookup / composition and its backward, with the collectives of the row-sharded step issued from inside
// the kernels:
//
//   lookup_compose_vec     each thread owns 8 consecutive columns of every algebra block of one query: it pulls the
//                          head row from its owner (peer loads over NVLink), composes the query and publishes the
//                          bf16 result with ONE 16-byte `multimem.st` through the NVSwitch multicast mapping of the
//                          query buffer (the all-gather of Q), or with one 16-byte store per destination rank when
//                          no multicast mapping exists.  The (h, r, data point) indices travel with the row.
//   compose_backward_owner the rank that owns a head row handles that query's backward: the query gradient is the
//                          sum of every rank's partial, fetched with `multimem.ld_reduce.add` (reduced inside the
//                          switch: the reduce-scatter of dQ) or by summing peer loads; chain rule; the row gradient
//                          is added to the local gradient shard, so no row gradient crosses the fabric.
//
// Entity row e lives on rank e % W at local row e / W.  Both kernels leave at once when the status word already
// holds an error (a timed-out barrier, a bad index), so that a rank whose peers are gone stops touching their memory.
// The reference has no counterpart: its lookups are `nn.Embedding` gathers on one device and its only collective is
// DDP's gradient all-reduce (dicee/models/base_model.py:371-383, dicee/trainer/torch_trainer_ddp.py:88).
#include "dice_b200.h"
#include "algebra.cuh"
#include "ptx_sm100.cuh"
#include "launch_pdl.cuh"

namespace dice {

// One 16-byte store to every GPU bound to the multicast object.
__device__ __forceinline__ void multimem_st_16(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
               "f"(__uint_as_float(v.w))
               : "memory");
}
// Sum over all GPUs bound to the multicast object of four consecutive floats (added inside the switch).
__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const void* mc_addr) {
  float4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w)
               : "l"(mc_addr)
               : "memory");
  return r;
}

template <int K>
__device__ __forceinline__ void load_blocks8(const float* row, int w, int j0, float (&v)[K][8]) {
#pragma unroll
  for (int a = 0; a < K; ++a) {
    const float4 lo = *reinterpret_cast<const float4*>(row + a * w + j0);
    const float4 hi = *reinterpret_cast<const float4*>(row + a * w + j0 + 4);
    v[a][0] = lo.x; v[a][1] = lo.y; v[a][2] = lo.z; v[a][3] = lo.w;
    v[a][4] = hi.x; v[a][5] = hi.y; v[a][6] = hi.z; v[a][7] = hi.w;
  }
}

// rh = normalised relation, nrm = the norm every element was divided by.
template <int K>
__device__ __forceinline__ void normalize_rel8(int mode, const float (&r)[K][8], float (&rh)[K][8],
                                               float (&nrm)[K][8]) {
#pragma unroll
  for (int a = 0; a < K; ++a)
#pragma unroll
    for (int u = 0; u < 8; ++u) { rh[a][u] = r[a][u]; nrm[a][u] = 1.f; }
  if (mode == NORM_ACROSS_BLOCKS) {
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      float s = 0.f;
#pragma unroll
      for (int a = 0; a < K; ++a) s += r[a][u] * r[a][u];
      const float n = sqrtf(s);
#pragma unroll
      for (int a = 0; a < K; ++a) { rh[a][u] = r[a][u] / n; nrm[a][u] = n; }
    }
  } else if (mode == NORM_CONSECUTIVE4) {   // groups of four consecutive columns of the row
#pragma unroll
    for (int a = 0; a < K; ++a)
#pragma unroll
      for (int g = 0; g < 8; g += 4) {
        float s = 0.f;
#pragma unroll
        for (int u = 0; u < 4; ++u) s += r[a][g + u] * r[a][g + u];
        const float n = fmaxf(sqrtf(s), 1e-12f);
#pragma unroll
        for (int u = 0; u < 4; ++u) { rh[a][g + u] = r[a][g + u] / n; nrm[a][g + u] = n; }
      }
  }
}

struct LookupVecParams {
  const long long* idx_h;        // [B] global entity ids of this rank's queries (entry i at idx_h[i * idx_stride])
  const long long* idx_r;        // [B] relation ids, same stride: a [B, 2] batch of (h, r) pairs is read in place
  int idx_stride;
  const long long* dp_src;       // [B] data-point ids (optional)
  const float* const* ent;       // [W] fp32 shard bases (peer pointers allowed)
  const float* rel;              // [R, D] replicated
  const float* coeff;            // Keci coefficient or null
  __nv_bfloat16* const* q_dst;   // [n_dst] unicast destinations of the bf16 query rows
  __nv_bfloat16* q_mc;           // multicast address of the query buffer, or null
  float* q_f32;                  // optional local fp32 copy [B, D]
  long long* const* ids_dst;     // [n_dst] index buffers laid out as h[ids_stride] | r[ids_stride] | dp[ids_stride]
  long long ids_stride;
  long long q_row_offset;        // first destination row of this rank's batch
  long long num_entities;
  int num_relations;
  int n_dst, B, D, W, norm_mode, additive;
  int* status;
};

template <int K>
__global__ void __launch_bounds__(256) lookup_compose_vec_kernel(const LookupVecParams p) {
  if (*p.status != 0) return;
  const int w = p.D / K;
  const int per_row = w >> 3;
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (tid >= static_cast<long long>(p.B) * per_row) return;
  const int i = static_cast<int>(tid / per_row);
  const int j0 = static_cast<int>(tid % per_row) << 3;
  const long long h = p.idx_h[static_cast<long long>(i) * p.idx_stride];
  const long long r_id = p.idx_r[static_cast<long long>(i) * p.idx_stride];
  if (h < 0 || h >= p.num_entities || r_id < 0 || r_id >= p.num_relations) {
    atomicCAS(p.status, 0, ST_BAD_INDEX);
    return;
  }
  const long long row = p.q_row_offset + i;
  if (j0 == 0 && p.ids_dst != nullptr) {
    const long long d = p.dp_src != nullptr ? p.dp_src[i] : 0;
    for (int k = 0; k < p.n_dst; ++k) {
      long long* dst = p.ids_dst[k];
      dst[row] = h;
      dst[p.ids_stride + row] = r_id;
      dst[2 * p.ids_stride + row] = d;
    }
  }
  const float* hrow = p.ent[h % p.W] + (h / p.W) * p.D;
  const float* rrow = p.rel + r_id * p.D;
  float hv[K][8], rv[K][8], rh[K][8], nrm[K][8];
  load_blocks8<K>(hrow, w, j0, hv);
  load_blocks8<K>(rrow, w, j0, rv);
  normalize_rel8<K>(p.norm_mode, rv, rh, nrm);
  if (p.coeff != nullptr) {  // Keci Cl(0,1): the vector part of head and relation is scaled by the coefficient
    const float c = *p.coeff;
#pragma unroll
    for (int u = 0; u < 8; ++u) { hv[K - 1][u] *= c; rh[K - 1][u] *= c; }
  }
#pragma unroll
  for (int k = 0; k < K; ++k) {
    float q[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      float acc = 0.f;
#pragma unroll
      for (int a = 0; a < K; ++a) acc = fmaf(Alg<K>::sgn(k, a) * hv[a][u], rh[Alg<K>::idx(k, a)][u], acc);
      q[u] = p.additive ? hv[k][u] + rh[k][u] : acc;
    }
    uint4 pk;
    __nv_bfloat162 b0 = __floats2bfloat162_rn(q[0], q[1]), b1 = __floats2bfloat162_rn(q[2], q[3]);
    __nv_bfloat162 b2 = __floats2bfloat162_rn(q[4], q[5]), b3 = __floats2bfloat162_rn(q[6], q[7]);
    pk.x = *reinterpret_cast<uint32_t*>(&b0);
    pk.y = *reinterpret_cast<uint32_t*>(&b1);
    pk.z = *reinterpret_cast<uint32_t*>(&b2);
    pk.w = *reinterpret_cast<uint32_t*>(&b3);
    const long long off = row * p.D + k * w + j0;
    if (p.q_mc != nullptr) {
      multimem_st_16(p.q_mc + off, pk);
    } else {
      for (int d = 0; d < p.n_dst; ++d) *reinterpret_cast<uint4*>(p.q_dst[d] + off) = pk;
    }
    if (p.q_f32 != nullptr) {
      float* qf = p.q_f32 + static_cast<long long>(i) * p.D + k * w + j0;
      *reinterpret_cast<float4*>(qf) = make_float4(q[0], q[1], q[2], q[3]);
      *reinterpret_cast<float4*>(qf + 4) = make_float4(q[4], q[5], q[6], q[7]);
    }
  }
}

struct BwdOwnerParams {
  const long long* idx_h;        // [n] global entity ids of the whole (global) batch (entry i at [i * idx_stride])
  const long long* idx_r;        // [n]
  int idx_stride;
  const float* ent_local;        // this rank's fp32 shard
  const float* rel;
  const float* coeff;
  const float* dq;               // [n, D] when the gradient is already complete locally (one rank)
  const float* const* dq_table;  // [n_dq] every rank's partial query gradients (peer pointers), or null
  const float* dq_mc;            // multicast address of the partial-gradient buffer, or null
  float* g_ent_local;            // [rows_local, D] gradient shard of this rank
  float* g_rel;                  // [R, D] this rank's partial relation gradient
  float* g_coeff;                // single float or null
  long long num_entities;
  int num_relations;
  int n, n_dq, D, W, rank, norm_mode, additive;
  int* status;
};

template <int K>
__global__ void __launch_bounds__(256) compose_backward_owner_kernel(const BwdOwnerParams p) {
  griddep_wait();
  griddep_launch();
  if (*p.status != 0) return;
  const int w = p.D / K;
  const int per_row = w >> 3;
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  float dc = 0.f;
  bool active = tid < static_cast<long long>(p.n) * per_row;
  int i = 0, j0 = 0;
  long long h = 0, r_id = 0;
  if (active) {
    i = static_cast<int>(tid / per_row);
    j0 = static_cast<int>(tid % per_row) << 3;
    h = p.idx_h[static_cast<long long>(i) * p.idx_stride];
    r_id = p.idx_r[static_cast<long long>(i) * p.idx_stride];
    if (h < 0 || h >= p.num_entities || r_id < 0 || r_id >= p.num_relations) {
      atomicCAS(p.status, 0, ST_BAD_INDEX);
      active = false;
    } else if (h % p.W != p.rank) {
      active = false;   // another rank owns this head row
    }
  }
  if (active) {
    const float* hrow = p.ent_local + (h / p.W) * p.D;
    const float* rrow = p.rel + r_id * p.D;
    float hv[K][8], rv[K][8], rh[K][8], nrm[K][8], dq[K][8], dh[K][8], drh[K][8];
    load_blocks8<K>(hrow, w, j0, hv);
    load_blocks8<K>(rrow, w, j0, rv);
    const long long qoff = static_cast<long long>(i) * p.D;
    if (p.dq_mc != nullptr) {          // reduce-scatter inside the switch
#pragma unroll
      for (int a = 0; a < K; ++a) {
        const float4 lo = multimem_ld_reduce_f32x4(p.dq_mc + qoff + a * w + j0);
        const float4 hi = multimem_ld_reduce_f32x4(p.dq_mc + qoff + a * w + j0 + 4);
        dq[a][0] = lo.x; dq[a][1] = lo.y; dq[a][2] = lo.z; dq[a][3] = lo.w;
        dq[a][4] = hi.x; dq[a][5] = hi.y; dq[a][6] = hi.z; dq[a][7] = hi.w;
      }
    } else if (p.dq_table != nullptr) {  // sum of the ranks' partial rows by peer loads
#pragma unroll
      for (int a = 0; a < K; ++a)
#pragma unroll
        for (int u = 0; u < 8; ++u) dq[a][u] = 0.f;
      for (int k = 0; k < p.n_dq; ++k) {
        float part[K][8];
        load_blocks8<K>(p.dq_table[k] + qoff, w, j0, part);
#pragma unroll
        for (int a = 0; a < K; ++a)
#pragma unroll
          for (int u = 0; u < 8; ++u) dq[a][u] += part[a][u];
      }
    } else {
      load_blocks8<K>(p.dq + qoff, w, j0, dq);
    }
    normalize_rel8<K>(p.norm_mode, rv, rh, nrm);
    float c = 1.f;
    if (p.coeff != nullptr) {
      c = *p.coeff;
#pragma unroll
      for (int u = 0; u < 8; ++u) { hv[K - 1][u] *= c; rh[K - 1][u] *= c; }
    }
#pragma unroll
    for (int a = 0; a < K; ++a)
#pragma unroll
      for (int u = 0; u < 8; ++u) { dh[a][u] = 0.f; drh[a][u] = 0.f; }
#pragma unroll
    for (int k = 0; k < K; ++k)
#pragma unroll
      for (int a = 0; a < K; ++a)
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float g = Alg<K>::sgn(k, a) * dq[k][u];
          dh[a][u] = fmaf(g, rh[Alg<K>::idx(k, a)][u], dh[a][u]);
          drh[Alg<K>::idx(k, a)][u] = fmaf(g, hv[a][u], drh[Alg<K>::idx(k, a)][u]);
        }
    if (p.additive) {
#pragma unroll
      for (int a = 0; a < K; ++a)
#pragma unroll
        for (int u = 0; u < 8; ++u) { dh[a][u] = dq[a][u]; drh[a][u] = dq[a][u]; }
    }
    if (p.coeff != nullptr) {
      // hv[K-1] = c * h_raw, rh[K-1] = c * r_raw  =>  d/dc collects both, the raw gradients pick up a factor c
#pragma unroll
      for (int u = 0; u < 8; ++u) {
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
      for (int u = 0; u < 8; ++u) {
        float dot = 0.f;
#pragma unroll
        for (int a = 0; a < K; ++a) dot += drh[a][u] * rh[a][u];
#pragma unroll
        for (int a = 0; a < K; ++a) drh[a][u] = (drh[a][u] - rh[a][u] * dot) / nrm[a][u];
      }
    } else if (p.norm_mode == NORM_CONSECUTIVE4) {
#pragma unroll
      for (int a = 0; a < K; ++a)
#pragma unroll
        for (int g = 0; g < 8; g += 4) {
          float dot = 0.f;
#pragma unroll
          for (int u = 0; u < 4; ++u) dot += drh[a][g + u] * rh[a][g + u];
#pragma unroll
          for (int u = 0; u < 4; ++u) drh[a][g + u] = (drh[a][g + u] - rh[a][g + u] * dot) / nrm[a][g + u];
        }
    }
    float* ge = p.g_ent_local + (h / p.W) * p.D;
    float* gr = p.g_rel + r_id * p.D;
#pragma unroll
    for (int a = 0; a < K; ++a) {
      red_add_v4(ge + a * w + j0, dh[a][0], dh[a][1], dh[a][2], dh[a][3]);
      red_add_v4(ge + a * w + j0 + 4, dh[a][4], dh[a][5], dh[a][6], dh[a][7]);
      red_add_v4(gr + a * w + j0, drh[a][0], drh[a][1], drh[a][2], drh[a][3]);
      red_add_v4(gr + a * w + j0 + 4, drh[a][4], drh[a][5], drh[a][6], drh[a][7]);
    }
  }
  if (p.g_coeff != nullptr) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dc += __shfl_xor_sync(0xffffffffu, dc, o);
    if ((threadIdx.x & 31) == 0 && dc != 0.f) atomicAdd(p.g_coeff, dc);
  }
}

// ------------------------------------------------------------------------------------ two-shot all-reduce + update
// Dense, replicated parameters (relation tables of models outside the sharded engines, convolution / linear / norm
// weights): the flat gradient buffers of all ranks live in the symmetric heap.  For one bucket [lo, hi) of the flat
// parameter vector every rank owns the slice lo + rank * len / W .. and, in ONE kernel,
//   1. reduce-scatter: sums that slice of every rank's gradient (multimem.ld_reduce through the switch, or W peer loads),
//   2. applies Adam / AdamW / SGD / ADOPT to its slice (moments are only ever touched for the slices a rank owns),
//   3. all-gather: stores the updated parameters into every rank's copy (multimem.st, or W peer stores).
// A rank therefore moves 1 / W of what a one-shot all-reduce would make it read.
struct BucketParams {
  float* const* p_dst;          // [W] flat parameter buffers of all ranks (peer pointers), used without multicast
  float* p_mc;                  // multicast address of the parameter buffer, or null
  const float* p_local;         // this rank's parameter buffer (read side)
  const float* const* g_src;    // [W] gradient buffers of all ranks, used without multicast
  const float* g_mc;            // multicast address of the gradient buffer, or null
  float* m;
  float* v;
  const long long* step;
  long long lo, hi;             // this rank's slice of the flat vector (multiples of 4)
  int W, kind;
  float lr, beta1, beta2, eps, weight_decay, grad_scale;
  const int* status;
};

__global__ void __launch_bounds__(256) bucket_reduce_update_kernel(const BucketParams p) {
  if (p.status != nullptr && *p.status != 0) return;
  const long long t = *p.step + 1;
  float inv_bc1 = 1.f, inv_sqrt_bc2 = 1.f;
  if (p.kind <= 1) {
    inv_bc1 = 1.f / (1.f - exp2f(static_cast<float>(t) * log2f(p.beta1)));
    inv_sqrt_bc2 = rsqrtf(1.f - exp2f(static_cast<float>(t) * log2f(p.beta2)));
  }
  const float clip = sqrtf(sqrtf(static_cast<float>(t - 1)));
  const bool first_step = (t == 1);
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 4;
  for (long long i = p.lo + (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * 4; i < p.hi; i += stride) {
    float4 g;
    if (p.g_mc != nullptr) {
      g = multimem_ld_reduce_f32x4(p.g_mc + i);
    } else {
      g = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int k = 0; k < p.W; ++k) {
        const float4 x = *reinterpret_cast<const float4*>(p.g_src[k] + i);
        g.x += x.x; g.y += x.y; g.z += x.z; g.w += x.w;
      }
    }
    g.x *= p.grad_scale; g.y *= p.grad_scale; g.z *= p.grad_scale; g.w *= p.grad_scale;
    float4 w = *reinterpret_cast<const float4*>(p.p_local + i);
    float4 m = make_float4(0.f, 0.f, 0.f, 0.f), v = m;
    if (p.kind != 2) {
      m = *reinterpret_cast<const float4*>(p.m + i);
      v = *reinterpret_cast<const float4*>(p.v + i);
    }
    float gg[4] = {g.x, g.y, g.z, g.w}, ww[4] = {w.x, w.y, w.z, w.w}, mm[4] = {m.x, m.y, m.z, m.w},
          vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float wd_g = (p.kind == 1) ? gg[u] : fmaf(p.weight_decay, ww[u], gg[u]);
      float wq = ww[u];
      if (p.kind == 1) wq *= 1.f - p.lr * p.weight_decay;
      if (p.kind == 0 || p.kind == 1) {
        mm[u] = fmaf(p.beta1, mm[u], (1.f - p.beta1) * wd_g);
        vv[u] = fmaf(p.beta2, vv[u], (1.f - p.beta2) * wd_g * wd_g);
        wq -= p.lr * inv_bc1 * mm[u] / (sqrtf(vv[u]) * inv_sqrt_bc2 + p.eps);
      } else if (p.kind == 2) {
        wq -= p.lr * wd_g;
      } else if (first_step) {   // ADOPT: the first step only seeds the second moment
        vv[u] = wd_g * wd_g;
      } else {
        float ng = wd_g / fmaxf(sqrtf(vv[u]), p.eps);
        ng = fminf(fmaxf(ng, -clip), clip);
        mm[u] += (1.f - p.beta1) * (ng - mm[u]);
        vv[u] = fmaf(p.beta2, vv[u], (1.f - p.beta2) * wd_g * wd_g);
        wq -= p.lr * mm[u];
      }
      ww[u] = wq;
    }
    if (p.kind != 2) {
      *reinterpret_cast<float4*>(p.m + i) = make_float4(mm[0], mm[1], mm[2], mm[3]);
      *reinterpret_cast<float4*>(p.v + i) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    }
    uint4 out;
    out.x = __float_as_uint(ww[0]); out.y = __float_as_uint(ww[1]);
    out.z = __float_as_uint(ww[2]); out.w = __float_as_uint(ww[3]);
    if (p.p_mc != nullptr) {
      multimem_st_16(p.p_mc + i, out);
    } else {
      for (int k = 0; k < p.W; ++k) *reinterpret_cast<uint4*>(p.p_dst[k] + i) = out;
    }
  }
}

template <int K>
static int launch_lookup_vec(const LookupVecParams& p, cudaStream_t s) {
  const long long n = static_cast<long long>(p.B) * (p.D / K / 8);
  lookup_compose_vec_kernel<K><<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
template <int K>
static int launch_bwd_owner(const BwdOwnerParams& p, cudaStream_t s) {
  const long long n = static_cast<long long>(p.n) * (p.D / K / 8);
  return launch_pdl(compose_backward_owner_kernel<K>, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0, s, p) ==
                 cudaSuccess
             ? 0
             : -4;
}

static int algebra_blocks(int model) {
  switch (model) {
    case 0: case 5: return 1;
    case 1: case 4: return 2;
    case 2: return 4;
    case 3: return 8;
    default: return 0;
  }
}

}  // namespace dice

using namespace dice;

// Returns 1 when the vectorised kernels cover (model, D): every algebra block must hold a multiple of 8 columns.
extern "C" int dice_lookup_vec_supported(int model, int D) {
  const int K = algebra_blocks(model);
  return (K > 0 && D % (8 * K) == 0) ? 1 : 0;
}

// model codes as in dice_lookup_compose.  idx_h / idx_r are read with stride idx_stride (1 for separate arrays; 2 with
// idx_r = idx_h + 1 reads a row-major [B, 2] batch of (h, r) pairs in place).  q_mc != null publishes the bf16 rows through the multicast mapping (all
// bound GPUs receive them at the same offset); otherwise they are stored to each of the n_dst buffers of q_dst.
// ids_dst (optional): n_dst index buffers receiving h, r and the data-point id of every row (three arrays, each
// ids_stride long).  ent / q_dst / ids_dst are device arrays of base pointers.
extern "C" int dice_lookup_compose_vec(int model, int normalize, const long long* idx_h, const long long* idx_r,
                                       int idx_stride, const long long* dp_src, const float* const* ent, int W,
                                       long long num_entities, int num_relations, const float* rel,
                                       const float* coeff, __nv_bfloat16* const* q_dst, int n_dst, void* q_mc,
                                       long long q_row_offset, float* q_f32, long long* const* ids_dst,
                                       long long ids_stride, int B, int D, int* status, void* stream) {
  if (B <= 0) return 0;
  if (!dice_lookup_vec_supported(model, D) || status == nullptr) return -6;
  if ((reinterpret_cast<uintptr_t>(rel) & 15) || (reinterpret_cast<uintptr_t>(q_mc) & 15) ||
      (reinterpret_cast<uintptr_t>(q_f32) & 15))
    return -5;
  LookupVecParams p{};
  p.idx_h = idx_h; p.idx_r = idx_r; p.idx_stride = idx_stride > 0 ? idx_stride : 1; p.dp_src = dp_src; p.ent = ent;
  p.rel = rel; p.coeff = nullptr;
  p.q_dst = q_dst; p.q_mc = static_cast<__nv_bfloat16*>(q_mc); p.q_f32 = q_f32; p.ids_dst = ids_dst;
  p.ids_stride = ids_stride; p.q_row_offset = q_row_offset; p.num_entities = num_entities;
  p.num_relations = num_relations; p.n_dst = n_dst; p.B = B; p.D = D; p.W = W; p.norm_mode = NORM_NONE;
  p.additive = 0; p.status = status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (model) {
    case 0: return launch_lookup_vec<1>(p, s);
    case 1: return launch_lookup_vec<2>(p, s);
    case 2: p.norm_mode = normalize ? NORM_CONSECUTIVE4 : NORM_NONE; return launch_lookup_vec<4>(p, s);
    case 3: p.norm_mode = normalize ? NORM_ACROSS_BLOCKS : NORM_NONE; return launch_lookup_vec<8>(p, s);
    case 4: p.coeff = coeff; return launch_lookup_vec<2>(p, s);
    case 5: p.additive = 1; return launch_lookup_vec<1>(p, s);
    default: return -6;
  }
}

// Backward of the composition for the queries whose head row this rank owns (h % W == rank); with W == 1 that is
// every query.  The query gradient comes from dq_mc (multimem.ld_reduce over all bound GPUs), else from the sum of
// the n_dq buffers of dq_table, else from dq.  Row gradients are added to g_ent_local (this rank's shard), relation
// gradients to g_rel (this rank's partial sum).
extern "C" int dice_compose_backward_owner(int model, int normalize, const long long* idx_h, const long long* idx_r,
                                           int idx_stride, const float* ent_local, int W, int rank, long long num_entities,
                                           int num_relations, const float* rel, const float* coeff, const float* dq,
                                           const float* const* dq_table, int n_dq, const void* dq_mc,
                                           float* g_ent_local, float* g_rel, float* g_coeff, int n, int D,
                                           int* status, void* stream) {
  if (n <= 0) return 0;
  if (!dice_lookup_vec_supported(model, D) || status == nullptr) return -6;
  if ((reinterpret_cast<uintptr_t>(rel) & 15) || (reinterpret_cast<uintptr_t>(dq) & 15) ||
      (reinterpret_cast<uintptr_t>(dq_mc) & 15) || (reinterpret_cast<uintptr_t>(ent_local) & 15) ||
      (reinterpret_cast<uintptr_t>(g_ent_local) & 15) || (reinterpret_cast<uintptr_t>(g_rel) & 15))
    return -5;
  BwdOwnerParams p{};
  p.idx_h = idx_h; p.idx_r = idx_r; p.idx_stride = idx_stride > 0 ? idx_stride : 1; p.ent_local = ent_local;
  p.rel = rel; p.coeff = nullptr; p.dq = dq;
  p.dq_table = dq_table; p.dq_mc = static_cast<const float*>(dq_mc); p.g_ent_local = g_ent_local; p.g_rel = g_rel;
  p.g_coeff = nullptr; p.num_entities = num_entities; p.num_relations = num_relations; p.n = n; p.n_dq = n_dq;
  p.D = D; p.W = W; p.rank = rank; p.norm_mode = NORM_NONE; p.additive = 0; p.status = status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (model) {
    case 0: return launch_bwd_owner<1>(p, s);
    case 1: return launch_bwd_owner<2>(p, s);
    case 2: p.norm_mode = normalize ? NORM_CONSECUTIVE4 : NORM_NONE; return launch_bwd_owner<4>(p, s);
    case 3: p.norm_mode = normalize ? NORM_ACROSS_BLOCKS : NORM_NONE; return launch_bwd_owner<8>(p, s);
    case 4: p.coeff = coeff; p.g_coeff = g_coeff; return launch_bwd_owner<2>(p, s);
    case 5: p.additive = 1; return launch_bwd_owner<1>(p, s);
    default: return -6;
  }
}

// Reduce-scatter of the partial query gradients on its own, in two launches.
//   dice_owned_rows    compacts the batch rows whose head entity this rank owns into a list (order irrelevant);
//   dice_dq_pull_owner sums, for every listed row, the W partial rows (one per rank, in dq_table) by peer loads and puts
//                      the sum in place of this rank's own partial row in dq_local.  Nobody else reads those rows (a
//                      peer pulls only the rows IT owns), so the update is in place.
// Both run on a graph branch beside the entity-role scoring launch, whose one CTA per SM (18 warps of 96 registers)
// leaves room for ONE more warp of at most 32 registers in each of the SM's four register partitions (measured: blocks
// of 256 threads do not start until the scoring CTA has left, a one-warp kernel does).  Hence blocks of 128 threads
// capped at 32 registers.  The pull is a persistent grid (16 bytes per work item, W independent loads in flight per
// thread); because the list holds owned rows only, every thread has loads in flight, which is what keeps NVLink busy
// at one resident block per SM.  The backward of the composition afterwards reads local memory only.
namespace dice {
// Kernels meant to run beside a scoring launch ask for the same shared-memory carveout as that launch (the maximum):
// an SM is not shared between kernels that want different carveouts.
template <typename Kern>
static void prefer_max_shared(Kern kern) {
  cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

__global__ void __launch_bounds__(128, 16) owned_rows_kernel(const long long* __restrict__ idx_h, int idx_stride, int n, int W,
                                                         int rank, long long num_entities, int* __restrict__ list,
                                                         int* __restrict__ count, int* status) {
  if (*status != 0) return;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  bool owned = false;
  if (i < n) {
    const long long h = idx_h[static_cast<long long>(i) * idx_stride];
    if (h < 0 || h >= num_entities) atomicCAS(status, 0, ST_BAD_INDEX);
    else owned = (h % W == rank);
  }
  const unsigned ballot = __ballot_sync(0xffffffffu, owned);
  const int lane = threadIdx.x & 31;
  int base = 0;
  if (lane == 0 && ballot != 0u) base = atomicAdd(count, __popc(ballot));
  base = __shfl_sync(0xffffffffu, base, 0);
  if (owned) list[base + __popc(ballot & ((1u << lane) - 1u))] = i;
}

__global__ void __launch_bounds__(128, 16) dq_pull_list_kernel(const int* __restrict__ list, const int* __restrict__ count,
                                                           const float* const* __restrict__ dq_table, int n_dq,
                                                           float* __restrict__ dq_local, int D, const int* status) {
  if (*status != 0) return;
  const int per_row = D >> 2;
  const long long total = static_cast<long long>(*count) * per_row;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long t = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; t < total; t += stride) {
    const int i = list[t / per_row];
    const size_t off = (static_cast<size_t>(i) * D >> 2) + static_cast<size_t>(t % per_row);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
    for (int k = 0; k < n_dq; ++k) {
      const float4 v = reinterpret_cast<const float4*>(dq_table[k])[off];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    reinterpret_cast<float4*>(dq_local)[off] = acc;
  }
}
}  // namespace dice

// list: int[n]; count: int[1], zeroed by the caller before the launch.
extern "C" int dice_owned_rows(const long long* idx_h, int idx_stride, int n, int W, int rank, long long num_entities,
                               int* list, int* count, int* status, void* stream) {
  if (n <= 0) return 0;
  if (status == nullptr || list == nullptr || count == nullptr || W < 1) return -5;
  dice::prefer_max_shared(dice::owned_rows_kernel);
  dice::owned_rows_kernel<<<(n + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      idx_h, idx_stride > 0 ? idx_stride : 1, n, W, rank, num_entities, list, count, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int dice_dq_pull_owner(const int* list, const int* count, const float* const* dq_table, int n_dq,
                                  float* dq_local, int D, int* status, void* stream) {
  if (n_dq <= 1) return 0;
  if (status == nullptr || dq_table == nullptr || list == nullptr || count == nullptr || (D & 3) ||
      (reinterpret_cast<uintptr_t>(dq_local) & 15))
    return -5;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  dice::prefer_max_shared(dice::dq_pull_list_kernel);
  dice::dq_pull_list_kernel<<<2 * sms, 128, 0, static_cast<cudaStream_t>(stream)>>>(list, count, dq_table, n_dq, dq_local,
                                                                                   D, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Two-shot all-reduce of one slice [lo, hi) of a flat gradient vector fused with the optimiser update of that slice
// and the broadcast of the updated parameters (see bucket_reduce_update_kernel).  lo, hi and every buffer must be
// 16-byte aligned.  g_mc / p_mc != null select the NVSwitch multicast path, otherwise g_src / p_dst (device arrays of
// W base pointers) are used.  grad_scale multiplies the summed gradient (1 / W for a mean over ranks).
extern "C" int dice_bucket_reduce_update(int kind, float* const* p_dst, void* p_mc, const float* p_local,
                                         const float* const* g_src, const void* g_mc, float* m, float* v,
                                         const long long* step, long long lo, long long hi, int W, float lr,
                                         float beta1, float beta2, float eps, float weight_decay, float grad_scale,
                                         const int* status, void* stream) {
  if (hi <= lo) return 0;
  if ((lo & 3) || (hi & 3)) return -5;
  if ((reinterpret_cast<uintptr_t>(p_mc) | reinterpret_cast<uintptr_t>(g_mc) | reinterpret_cast<uintptr_t>(p_local) |
       reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v)) & 15)
    return -5;
  BucketParams p{};
  p.p_dst = p_dst; p.p_mc = static_cast<float*>(p_mc); p.p_local = p_local; p.g_src = g_src;
  p.g_mc = static_cast<const float*>(g_mc); p.m = m; p.v = v; p.step = step; p.lo = lo; p.hi = hi; p.W = W;
  p.kind = kind; p.lr = lr; p.beta1 = beta1; p.beta2 = beta2; p.eps = eps; p.weight_decay = weight_decay;
  p.grad_scale = grad_scale; p.status = status;
  const long long n4 = (hi - lo) >> 2;
  long long blocks = (n4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  bucket_reduce_update_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
