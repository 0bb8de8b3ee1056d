// Kernels of the sampled-candidate training steps (negative sampling, 1vsSample, KvsSample):
//
//   dice_neg_sample      corrupted triples + labels generated on the device from a counter-based generator
//   dice_uniform_int     uniform integers in [0, high)
//   dice_candidate_bce   scores of each query against its own list of candidate entities, BCE-with-logits loss,
//                        and the gradients w.r.t. the query vectors and the candidate rows, in one pass
//
// The query vectors come from dice_lookup_compose (any of its algebras) and their gradient goes back through
// dice_compose_backward, so one scoring kernel serves every model of the bilinear family plus the translation model.
#include "dice_b200.h"
#include "ptx_sm100.cuh"

namespace dice {
namespace triple {

// ------------------------------------------------------------------------------------ Philox-4x32-10
struct Philox {
  uint32_t key[2];
  __device__ __forceinline__ Philox(unsigned long long seed) {
    key[0] = static_cast<uint32_t>(seed);
    key[1] = static_cast<uint32_t>(seed >> 32);
  }
  __device__ __forceinline__ uint4 operator()(unsigned long long counter, unsigned long long stream) const {
    uint32_t c0 = static_cast<uint32_t>(counter), c1 = static_cast<uint32_t>(counter >> 32);
    uint32_t c2 = static_cast<uint32_t>(stream), c3 = static_cast<uint32_t>(stream >> 32);
    uint32_t k0 = key[0], k1 = key[1];
#pragma unroll
    for (int r = 0; r < 10; ++r) {
      const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
      const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
      const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
      c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
      k0 += 0x9E3779B9u;
      k1 += 0xBB67AE85u;
    }
    return make_uint4(c0, c1, c2, c3);
  }
};

// Maps 64 random bits to [0, high) by the multiply-high reduction (bias below high / 2^64).
__device__ __forceinline__ long long bounded(uint32_t a, uint32_t b, long long high) {
  const unsigned long long x = (static_cast<unsigned long long>(a) << 32) | b;
  return static_cast<long long>(__umul64hi(x, static_cast<unsigned long long>(high)));
}

__global__ void uniform_int_kernel(long long* __restrict__ out, long long n, long long high, unsigned long long seed,
                                   unsigned long long offset, const long long* __restrict__ step_ptr,
                                   long long out_stride, long long row_len) {
  const Philox rng(seed);
  if (step_ptr != nullptr) offset += static_cast<unsigned long long>(*step_ptr);
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; 2 * i < n; i += stride) {
    const uint4 r = rng(static_cast<unsigned long long>(i), offset);
    // element j of the flat sequence lands at row j / row_len, column j % row_len of a matrix with row stride
    // out_stride (row_len == out_stride == n for a plain vector)
    const long long j0 = 2 * i, j1 = 2 * i + 1;
    out[(j0 / row_len) * out_stride + j0 % row_len] = bounded(r.x, r.y, high);
    if (j1 < n) out[(j1 / row_len) * out_stride + j1 % row_len] = bounded(r.z, r.w, high);
  }
}

// Output layout: rows [0, B) are the positives, row B + j * B + i is the j-th corruption of positive i.
// mode 0: one coin per call decides whether all heads or all tails are replaced; mode 1: one coin per negative.
// step_ptr (optional) is added to offset on the device, so a captured launch draws new samples at every replay.
__global__ void neg_sample_kernel(const long long* __restrict__ pos, int B, int k, long long num_entities,
                                  unsigned long long seed, unsigned long long offset,
                                  const long long* __restrict__ step_ptr, int mode, float label_pos, float label_neg,
                                  long long* __restrict__ x, long long* __restrict__ h_out,
                                  long long* __restrict__ r_out, long long* __restrict__ t_out,
                                  float* __restrict__ y) {
  const Philox rng(seed);
  if (step_ptr != nullptr) offset += static_cast<unsigned long long>(*step_ptr);
  const bool batch_heads = (rng(~0ull, offset).x & 1u) != 0u;
  const long long total = static_cast<long long>(B) * (1 + k);
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long n = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; n < total; n += stride) {
    const int i = static_cast<int>(n % B);
    long long h = pos[3 * i], r = pos[3 * i + 1], t = pos[3 * i + 2];
    float label = label_pos;
    if (n >= B) {
      const uint4 u = rng(static_cast<unsigned long long>(n), offset);
      const long long e = bounded(u.x, u.y, num_entities);
      const bool heads = mode == 0 ? batch_heads : (u.z & 1u) != 0u;
      if (heads) h = e; else t = e;
      label = label_neg;
    }
    if (x != nullptr) {
      x[3 * n] = h;
      x[3 * n + 1] = r;
      x[3 * n + 2] = t;
    }
    if (h_out != nullptr) {
      h_out[n] = h;
      r_out[n] = r;
      t_out[n] = t;
    }
    y[n] = label;
  }
}

// ------------------------------------------------------------------------------------ candidate scoring
struct CandParams {
  const float* q;             // [N, D] query vectors (fp32)
  const long long* cand;      // candidate entity ids: entry (n, c) at cand[n * cand_stride + c * cand_step]
  long long cand_stride, cand_step;
  int C;                      // candidates per query
  const float* labels;        // [N, C] targets in [0, 1]
  const float* const* ent;    // [W] fp32 entity shards, entity e lives in shard e % W at row e / W
  float* const* g_ent;        // [W] gradient shards (red.add); null = forward only
  unsigned char* const* touched;  // optional [W] per-row flags of the gradient shards
  float* dq;                  // [N, D] gradient w.r.t. q (written, not accumulated); null = forward only
  float* scores;              // [N, C] or null
  double* loss;               // accumulator of sum(BCE) * scale, or null
  float scale;                // 1 / (N * C) for a mean-reduced loss
  float margin;               // distance kind: score = margin - ||q + eps - t||
  float eps;
  int N, D, W, kind;          // kind 0: dot product, 1: negative Euclidean distance
  long long num_entities;     // > 0 (with status): candidate ids outside [0, num_entities) are reported and replaced
  int* status;                // by entity 0, whose contribution is then dropped
};

// One warp per query: the query stays in registers while its candidates stream through, CH candidate rows in flight
// at a time (their loads are all issued before the first dot product is reduced).
template <int NV, int CH>  // float4 chunks per lane (D <= NV * 128), candidates in flight
__global__ void __launch_bounds__(256) candidate_bce_kernel(const CandParams p) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  double loss_local = 0.0;
  for (int n = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; n < p.N; n += warps) {
    float4 qv[NV], dqv[NV];
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int d = (v * 32 + lane) * 4;
      qv[v] = d < p.D ? *reinterpret_cast<const float4*>(p.q + static_cast<size_t>(n) * p.D + d)
                      : make_float4(0.f, 0.f, 0.f, 0.f);
      dqv[v] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int c0 = 0; c0 < p.C; c0 += CH) {
      long long ent_id[CH];
      float4 tv[CH][NV];
      float acc[CH];
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        const int c = c0 + j < p.C ? c0 + j : c0;   // the tail of the list repeats a valid candidate; results are dropped
        ent_id[j] = p.cand[n * p.cand_stride + c * p.cand_step];
        if (p.num_entities > 0 && (ent_id[j] < 0 || ent_id[j] >= p.num_entities)) {
          if (lane == 0 && p.status != nullptr) atomicCAS(p.status, 0, dice::ST_BAD_INDEX);
          ent_id[j] = -1;
        }
      }
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        const long long e_safe = ent_id[j] < 0 ? 0 : ent_id[j];
        const float* trow = p.ent[e_safe % p.W] + static_cast<size_t>(e_safe / p.W) * p.D;
#pragma unroll
        for (int v = 0; v < NV; ++v) {
          const int d = (v * 32 + lane) * 4;
          tv[j][v] = d < p.D ? *reinterpret_cast<const float4*>(trow + d) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        float a = 0.f;
#pragma unroll
        for (int v = 0; v < NV; ++v) {
          const int d = (v * 32 + lane) * 4;
          if (d < p.D) {
            if (p.kind == 0) {
              a = fmaf(qv[v].x, tv[j][v].x, a); a = fmaf(qv[v].y, tv[j][v].y, a);
              a = fmaf(qv[v].z, tv[j][v].z, a); a = fmaf(qv[v].w, tv[j][v].w, a);
            } else {
              const float x0 = qv[v].x + p.eps - tv[j][v].x, x1 = qv[v].y + p.eps - tv[j][v].y;
              const float x2 = qv[v].z + p.eps - tv[j][v].z, x3 = qv[v].w + p.eps - tv[j][v].w;
              a += x0 * x0 + x1 * x1 + x2 * x2 + x3 * x3;
            }
          }
        }
        acc[j] = a;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
        for (int j = 0; j < CH; ++j) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
      }
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        const int c = c0 + j;
        if (c >= p.C || ent_id[j] < 0) continue;
        float dist = 0.f;
        float s = acc[j];
        if (p.kind == 1) {
          dist = sqrtf(acc[j]);
          s = p.margin - dist;
        }
        const size_t flat = static_cast<size_t>(n) * p.C + c;
        if (lane == 0 && p.scores != nullptr) p.scores[flat] = s;
        if (p.labels == nullptr) continue;
        const float y = p.labels[flat];
        if (lane == 0) loss_local += static_cast<double>(fmaxf(s, 0.f) - s * y + log1pf(expf(-fabsf(s))));
        if (p.dq == nullptr) continue;
        float g = (1.f / (1.f + expf(-s)) - y) * p.scale;  // dL/ds
        const long long e = ent_id[j];
        float* grow = p.g_ent[e % p.W] + static_cast<size_t>(e / p.W) * p.D;
        if (p.touched != nullptr && lane == 0) p.touched[e % p.W][e / p.W] = 1;
        if (p.kind == 0) {
#pragma unroll
          for (int v = 0; v < NV; ++v) {
            const int d = (v * 32 + lane) * 4;
            if (d < p.D) {
              dqv[v].x = fmaf(g, tv[j][v].x, dqv[v].x); dqv[v].y = fmaf(g, tv[j][v].y, dqv[v].y);
              dqv[v].z = fmaf(g, tv[j][v].z, dqv[v].z); dqv[v].w = fmaf(g, tv[j][v].w, dqv[v].w);
              red_add_v4(grow + d, g * qv[v].x, g * qv[v].y, g * qv[v].z, g * qv[v].w);
            }
          }
        } else {
          // s = margin - dist, d dist / d q = (q + eps - t) / dist
          g = dist > 0.f ? -g / dist : 0.f;
#pragma unroll
          for (int v = 0; v < NV; ++v) {
            const int d = (v * 32 + lane) * 4;
            if (d < p.D) {
              const float x0 = g * (qv[v].x + p.eps - tv[j][v].x), x1 = g * (qv[v].y + p.eps - tv[j][v].y);
              const float x2 = g * (qv[v].z + p.eps - tv[j][v].z), x3 = g * (qv[v].w + p.eps - tv[j][v].w);
              dqv[v].x += x0; dqv[v].y += x1; dqv[v].z += x2; dqv[v].w += x3;
              red_add_v4(grow + d, -x0, -x1, -x2, -x3);
            }
          }
        }
      }
    }
    if (p.dq != nullptr) {
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        const int d = (v * 32 + lane) * 4;
        if (d < p.D) *reinterpret_cast<float4*>(p.dq + static_cast<size_t>(n) * p.D + d) = dqv[v];
      }
    }
  }
  if (p.loss != nullptr && lane == 0 && loss_local != 0.0) atomicAdd(p.loss, loss_local * p.scale);
}

// ------------------------------------------------------------------------------------ row-wise sparse optimiser
// Only rows that received a gradient are touched: their moments decay lazily (as in torch.optim.SparseAdam), the
// bias correction uses the global step.  The gradient row and the flag are cleared on the way out.
struct SparseOptParams {
  float* __restrict__ param;
  float* __restrict__ grad;
  float* __restrict__ m;
  float* __restrict__ v;
  __nv_bfloat16* __restrict__ shadow;      // optional bf16 copy of the parameters, refreshed for updated rows
  unsigned char* __restrict__ touched;
  long long rows;
  int D, kind;                // 0 Adam, 1 AdamW, 2 SGD
  const long long* step;      // completed steps (the update uses step + 1)
  float lr, beta1, beta2, eps, weight_decay;
};

__global__ void __launch_bounds__(256) sparse_rows_optimizer_kernel(const SparseOptParams p) {
  // A block takes 256 consecutive rows at a time: one flag per thread, the flagged rows are compacted into shared
  // memory in row order and dealt to the 8 warps round-robin, so the warps of a block (and neighbouring blocks) work
  // on neighbouring rows at the same moment and DRAM pages are used whole.
  __shared__ unsigned char list[256];
  __shared__ int warp_count[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float t = static_cast<float>(*p.step + 1);
  float inv_bc1 = 1.f, inv_sqrt_bc2 = 1.f;
  if (p.kind != 2) {
    inv_bc1 = 1.f / (1.f - exp2f(t * log2f(p.beta1)));
    inv_sqrt_bc2 = rsqrtf(1.f - exp2f(t * log2f(p.beta2)));
  }
  for (long long base = static_cast<long long>(blockIdx.x) * 256; base < p.rows;
       base += static_cast<long long>(gridDim.x) * 256) {
    const long long mine = base + threadIdx.x;
    const bool flag = mine < p.rows && p.touched[mine] != 0;
    if (flag) p.touched[mine] = 0;
    const unsigned int bits = __ballot_sync(0xffffffffu, flag);
    if (lane == 0) warp_count[warp] = __popc(bits);
    __syncthreads();
    int before = 0, total = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const int c = warp_count[w];
      if (w < warp) before += c;
      total += c;
    }
    if (flag) list[before + __popc(bits & ((1u << lane) - 1u))] = static_cast<unsigned char>(threadIdx.x);
    __syncthreads();
    // four rows per warp are in flight at a time: all their loads are issued before the first store
    constexpr int R = 4;
    for (int i0 = warp; i0 < total; i0 += 8 * R) {
      for (int d = lane * 4; d < p.D; d += 128) {
        size_t off[R];
        float4 g4[R], w4[R], m4[R], v4[R];
#pragma unroll
        for (int j = 0; j < R; ++j) {
          const int i = i0 + 8 * j;
          off[j] = static_cast<size_t>(base + list[i < total ? i : i0]) * p.D + d;
          g4[j] = *reinterpret_cast<const float4*>(p.grad + off[j]);
          w4[j] = *reinterpret_cast<const float4*>(p.param + off[j]);
          m4[j] = make_float4(0.f, 0.f, 0.f, 0.f);
          v4[j] = m4[j];
          if (p.kind != 2) {
            m4[j] = *reinterpret_cast<const float4*>(p.m + off[j]);
            v4[j] = *reinterpret_cast<const float4*>(p.v + off[j]);
          }
        }
#pragma unroll
        for (int j = 0; j < R; ++j) {
          if (i0 + 8 * j >= total) continue;
          *reinterpret_cast<float4*>(p.grad + off[j]) = make_float4(0.f, 0.f, 0.f, 0.f);
          float gp[4] = {g4[j].x, g4[j].y, g4[j].z, g4[j].w};
          float wp[4] = {w4[j].x, w4[j].y, w4[j].z, w4[j].w};
          if (p.kind == 2) {
#pragma unroll
            for (int u = 0; u < 4; ++u) wp[u] -= p.lr * fmaf(p.weight_decay, wp[u], gp[u]);
          } else {
            float mp[4] = {m4[j].x, m4[j].y, m4[j].z, m4[j].w};
            float vp[4] = {v4[j].x, v4[j].y, v4[j].z, v4[j].w};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              float gu = gp[u];
              if (p.kind == 0) gu = fmaf(p.weight_decay, wp[u], gu);
              else wp[u] *= 1.f - p.lr * p.weight_decay;
              mp[u] = fmaf(p.beta1, mp[u], (1.f - p.beta1) * gu);
              vp[u] = fmaf(p.beta2, vp[u], (1.f - p.beta2) * gu * gu);
              wp[u] -= p.lr * inv_bc1 * mp[u] / (sqrtf(vp[u]) * inv_sqrt_bc2 + p.eps);
            }
            *reinterpret_cast<float4*>(p.m + off[j]) = make_float4(mp[0], mp[1], mp[2], mp[3]);
            *reinterpret_cast<float4*>(p.v + off[j]) = make_float4(vp[0], vp[1], vp[2], vp[3]);
          }
          *reinterpret_cast<float4*>(p.param + off[j]) = make_float4(wp[0], wp[1], wp[2], wp[3]);
          if (p.shadow != nullptr) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(wp[0], wp[1]), hi = __floats2bfloat162_rn(wp[2], wp[3]);
            uint2 pk = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
            *reinterpret_cast<uint2*>(p.shadow + off[j]) = pk;
          }
        }
      }
    }
    __syncthreads();  // the list is rebuilt for the next chunk
  }
}

}  // namespace triple
}  // namespace dice

// Row-wise sparse update of a [rows, D] table: rows with touched[row] != 0 are updated from grad (then grad row and
// flag are cleared), all other rows are left alone.  kind: 0 Adam, 1 AdamW, 2 SGD.  D must be a multiple of 4.
extern "C" int dice_sparse_rows_optimizer(int kind, float* param, float* grad, float* m, float* v, void* shadow,
                                          unsigned char* touched, long long rows, int D, const long long* step,
                                          float lr, float beta1, float beta2, float eps, float weight_decay,
                                          void* stream) {
  using namespace dice::triple;
  if (rows <= 0) return 0;
  if (D % 4 || kind < 0 || kind > 2) return -6;
  SparseOptParams p{param, grad, m, v, static_cast<__nv_bfloat16*>(shadow), touched, rows, D, kind, step, lr, beta1,
                    beta2, eps, weight_decay};
  long long blocks = (rows + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  sparse_rows_optimizer_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// With row_len > 0 the n draws fill a [n / row_len, row_len] block of a matrix whose rows are out_stride apart
// (e.g. the negative columns of a candidate matrix); step_ptr (optional, device) is added to offset.
extern "C" int dice_uniform_int(long long* out, long long n, long long high, unsigned long long seed,
                                unsigned long long offset, const long long* step_ptr, long long out_stride,
                                long long row_len, void* stream) {
  if (n <= 0) return 0;
  if (high <= 0) return -6;
  if (row_len <= 0) { row_len = n; out_stride = n; }
  long long blocks = ((n + 1) / 2 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  dice::triple::uniform_int_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      out, n, high, seed, offset, step_ptr, out_stride, row_len);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// pos: [B, 3] int64 triples; outputs for N = B * (1 + k) rows: x [N, 3] (optional) and / or the columns h, r, t [N]
// (optional, all three or none), y [N] fp32.  The same (seed, offset + *step_ptr) reproduces the same corruptions.
extern "C" int dice_neg_sample(const long long* pos, int B, int k, long long num_entities, unsigned long long seed,
                               unsigned long long offset, const long long* step_ptr, int mode, float label_pos,
                               float label_neg, long long* x, long long* h, long long* r, long long* t, float* y,
                               void* stream) {
  if (B <= 0) return 0;
  if (k < 0 || num_entities <= 0) return -6;
  long long blocks = (static_cast<long long>(B) * (1 + k) + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  dice::triple::neg_sample_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      pos, B, k, num_entities, seed, offset, step_ptr, mode, label_pos, label_neg, x, h, r, t, y);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Scores query n against candidates cand[n * cand_stride + c * cand_step], c < C.  With labels it accumulates the
// BCE-with-logits loss (times scale) and, when dq / g_ent are given, writes dq and adds the candidate-row gradients.
// D must be a multiple of 4 and at most 512; q, dq and the entity shards must be 16-byte aligned.
extern "C" int dice_candidate_bce(const float* q, const long long* cand, long long cand_stride, long long cand_step,
                                  int C, const float* labels, const float* const* ent, float* const* g_ent, float* dq,
                                  float* scores, double* loss, float scale, int kind, float margin, float eps, int N,
                                  int D, int W, unsigned char* const* touched, long long num_entities, int* status,
                                  void* stream) {
  using namespace dice::triple;
  if (N <= 0 || C <= 0) return 0;
  if (D % 4 || D > 512 || W <= 0) return -6;
  if ((dq == nullptr) != (g_ent == nullptr)) return -6;
  CandParams p{q, cand, cand_stride, cand_step, C, labels, ent, g_ent, touched, dq, scores, loss, scale, margin, eps,
               N, D, W, kind, num_entities, status};
  const int threads = 256;
  long long blocks = (static_cast<long long>(N) * 32 + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (D <= 128) candidate_bce_kernel<1, 4><<<static_cast<unsigned>(blocks), threads, 0, s>>>(p);
  else if (D <= 256) candidate_bce_kernel<2, 4><<<static_cast<unsigned>(blocks), threads, 0, s>>>(p);
  else candidate_bce_kernel<4, 2><<<static_cast<unsigned>(blocks), threads, 0, s>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
