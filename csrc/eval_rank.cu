// Fused link-prediction ranking / top-k kernel for sm_100a (tcgen05 + TMEM + TMA) and its sparse companion.
//
// dice_eval_rank:   for queries X [x_rows, D] and entity rows Y [y_rows, D] (bf16, row-major) the tensor cores
//                   produce S = X · Yᵀ tile by tile in TMEM; the epilogue never stores S.  It counts, per query row,
//                   the entities whose score exceeds that row's target score (the dense part of
//                   rank = 1 + #greater − #filtered greater) and, optionally, keeps a running top-k per row.
// dice_eval_sparse: gather-dots for the sparse part: the target score of each query and the number of *filtered*
//                   entities (a CSR list per query) that beat it.
//
// The same CTA structure as the training kernel is used (warp 0 TMA producer, warp 1 MMA issuer, warps 2..9
// epilogue, one persistent CTA per SM over a contiguous range of (x-tile, y-tile) pairs) but there is no second
// GEMM, so all 512 TMEM columns hold four S buffers.  Every wait is bounded and reports through the status word.
#include "dice_b200.h"
#include "ptx_sm100.cuh"
#include "tile_map.cuh"
#include "tma_host.cuh"

#include <math_constants.h>

namespace dice {

namespace evalk {

constexpr int BLOCK_X = 128;
constexpr int BLOCK_Y = 128;
constexpr int SLAB_BYTES = 128 * 128;
constexpr int NUM_THREADS = 320;
constexpr int NUM_EPI_WARPS = 8;
constexpr int NBUF = 4;       // S buffers in TMEM
constexpr int KMAX = 32;      // largest k of the in-kernel top-k

struct EvalParams {
  const float* target;     // [x_rows] score of the true entity of each query (columns beat it when s > target)
  const int* target_idx;   // [x_rows] column of the true entity (never counted); may be null
  const float* col_bias;   // [y_rows] added to every score of that column; may be null
  int* greater;            // [x_rows] += number of columns with s > target
  int* status;
  int x_rows, y_rows, nx_tiles, ny_tiles;
  TileMap map;             // visiting order of the (x tile, y tile) pairs
  int y_offset, y_stride;  // global id of column c is y_offset + c * y_stride (contiguous or cyclic row shards)
  // top-k (TOPK variants): every (segment, row, half) appends its k best to the row's candidate list
  int k;
  int cand_cap;            // capacity of a row's candidate list (entries)
  float* cand_score;       // [x_rows, cand_cap], pre-filled with -inf
  int* cand_idx;           // [x_rows, cand_cap], pre-filled with -1
  int* cand_count;         // [x_rows], zero-initialised
  float* row_floor;        // [x_rows], pre-filled with -inf: best known lower bound of each row's k-th best score,
                           // published by finished segments so that later segments start with a tight threshold
  // band mode (BAND variants): scores within +-margin[row] of the target are not decided here; their (row, entity)
  // pairs are appended to a list for an exact second pass, only scores above target + margin are counted
  const float* margin;     // [x_rows]
  int* band_rows;          // [band_cap]
  int* band_cols;          // [band_cap] global entity ids
  unsigned long long* band_count;
  long long band_cap;
};

template <int D>
struct Cfg {
  static constexpr int NSLAB = D / 64;
  static constexpr int TILE_BYTES = NSLAB * SLAB_BYTES;
  static constexpr int NSTAGE = (D == 256) ? 2 : 4;
  static constexpr int SMEM_BYTES = TILE_BYTES * (1 + NSTAGE) + 1024 + 512;
};

__device__ __forceinline__ void atomic_max_float(float* addr, float v) {
  if (v >= 0.f) atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v));
  else atomicMin(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v));
}

template <int D, int MODE>  // 0 count, 1 count + running top-k, 2 count with an undecided band, 3 collect above floor
__global__ void __launch_bounds__(NUM_THREADS, 1)
eval_rank_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_y,
                 const EvalParams p) {
  using C = Cfg<D>;
  constexpr bool TOPK = MODE == 1;
  constexpr bool BAND = MODE == 2;
  constexpr bool COLLECT = MODE == 3;  // every score >= row_floor[row] is appended to the row's candidate list
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sX = smem;
  uint8_t* sY = smem + C::TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::TILE_BYTES * (1 + C::NSTAGE));
  uint64_t* x_full = bars + 0;
  uint64_t* x_empty = bars + 1;
  uint64_t* s_full = bars + 2;    // [NBUF]
  uint64_t* s_empty = bars + 6;   // [NBUF]
  uint64_t* y_full = bars + 10;   // [NSTAGE]
  uint64_t* y_empty = bars + 14;  // [NSTAGE]
  uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(bars + 18);
  volatile int* s_abort = reinterpret_cast<volatile int*>(bars + 19);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = static_cast<long long>(p.nx_tiles) * p.ny_tiles;
  const long long w_begin = total * blockIdx.x / gridDim.x;
  const long long w_end = total * (blockIdx.x + 1) / gridDim.x;

  if (threadIdx.x == 0) {
    mbar_init(x_full, 1);
    mbar_init(x_empty, 1);
    for (int i = 0; i < NBUF; ++i) {
      mbar_init(s_full + i, 1);
      mbar_init(s_empty + i, NUM_EPI_WARPS);
    }
    for (int i = 0; i < C::NSTAGE; ++i) {
      mbar_init(y_full + i, 1);
      mbar_init(y_empty + i, 1);
    }
    *reinterpret_cast<volatile uint64_t*>(bars + 19) = 0;  // abort flag and an always-zero word next to it
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_smem, 512);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_x);
    tma_prefetch_desc(&tmap_y);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_smem;

  auto fail = [&](int code) {
    atomicCAS(p.status, 0, code);
    *s_abort = 1;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------------- TMA producer
    if (lane == 0) {
      uint32_t ycount = 0, seg = 0, x_loads = 0;
      for (long long w = w_begin; w < w_end && !*s_abort;) {
        int x, y0, run;
        p.map.locate(w, x, y0, run);
        const int n = static_cast<int>(min(static_cast<long long>(run), w_end - w));
        if (!mbar_wait_bounded(x_empty, (seg & 1) ^ 1, s_abort)) { fail(ST_TIMEOUT_PRODUCER); break; }
        mbar_arrive_expect_tx(x_full, C::TILE_BYTES);
        for (int s = 0; s < C::NSLAB; ++s) tma_load_2d(sX + s * SLAB_BYTES, &tmap_x, s * 64, x * BLOCK_X, x_full);
        ++x_loads;
        bool ok = true;
        for (int t = 0; t < n; ++t, ++ycount) {
          const uint32_t st = ycount % C::NSTAGE;
          if (!mbar_wait_bounded(y_empty + st, ((ycount / C::NSTAGE) & 1) ^ 1, s_abort)) { ok = false; break; }
          mbar_arrive_expect_tx(y_full + st, C::TILE_BYTES);
          uint8_t* dst = sY + st * C::TILE_BYTES;
          for (int s = 0; s < C::NSLAB; ++s)
            tma_load_2d(dst + s * SLAB_BYTES, &tmap_y, s * 64, (y0 + t) * BLOCK_Y, y_full + st);
        }
        if (!ok) { fail(ST_TIMEOUT_PRODUCER); break; }
        w += n;
        ++seg;
      }
      if (*s_abort) {  // every copy issued by this thread must land before the CTA exits
        bool drained = true;
        if (x_loads > 0) drained &= mbar_wait_bounded(x_full, (x_loads - 1) & 1, s_abort + 1, 1u << 20);
        for (uint32_t i = 0; i < C::NSTAGE && i < ycount; ++i) {
          const uint32_t last = ycount - 1 - i;
          drained &= mbar_wait_bounded(y_full + (last % C::NSTAGE), (last / C::NSTAGE) & 1, s_abort + 1, 1u << 20);
        }
        if (!drained) atomicExch(p.status, ST_TIMEOUT_DRAIN);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t IDESC = make_idesc_bf16(BLOCK_X, BLOCK_Y, 0, 0);
      const uint32_t sx_addr = smem_u32(sX);
      uint32_t g = 0, seg = 0;
      bool ok = true;
      for (long long w = w_begin; w < w_end && ok && !*s_abort;) {
        int x, y0, run;
        p.map.locate(w, x, y0, run);
        const int n = static_cast<int>(min(static_cast<long long>(run), w_end - w));
        if (!mbar_wait_bounded(x_full, seg & 1, s_abort)) { ok = false; break; }
        for (int t = 0; t < n; ++t, ++g) {
          const uint32_t st = g % C::NSTAGE;
          const uint32_t b = g % NBUF;
          if (!mbar_wait_bounded(y_full + st, (g / C::NSTAGE) & 1, s_abort)) { ok = false; break; }
          if (!mbar_wait_bounded(s_empty + b, ((g / NBUF) & 1) ^ 1, s_abort)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sy_addr = smem_u32(sY + st * C::TILE_BYTES);
          const uint32_t d_tmem = tmem_base + b * BLOCK_Y;
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint32_t off = (k >> 2) * SLAB_BYTES + (k & 3) * 32;
            mma_ss(d_tmem, make_sw128_desc(sx_addr + off, 16, 1024), make_sw128_desc(sy_addr + off, 16, 1024), IDESC,
                   k > 0 ? 1u : 0u);
          }
          tc_commit(y_empty + st);
          tc_commit(s_full + b);
          if (t + 1 == n) tc_commit(x_empty);
        }
        w += n;
        ++seg;
      }
      if (!ok) fail(ST_TIMEOUT_MMA);
    }
  } else {
    // ------------------------------------------------------------------------- epilogue warps
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    const int row = quarter * 32 + lane;
    uint32_t g = 0;
    bool ok = true;
    float top_s[TOPK ? KMAX : 1];
    int top_i[TOPK ? KMAX : 1];

    for (long long w = w_begin; w < w_end && ok && !*s_abort;) {
      int x, y0, run;
      p.map.locate(w, x, y0, run);
      const int n = static_cast<int>(min(static_cast<long long>(run), w_end - w));
      const int x_global = x * BLOCK_X + row;
      const bool valid_x = x_global < p.x_rows;
      const float tgt = (valid_x && p.target != nullptr) ? p.target[x_global] : CUDART_INF_F;
      int tgt_col = -1;
      if (valid_x && p.target_idx != nullptr) {
        const int rel_id = p.target_idx[x_global] - p.y_offset;
        if (rel_id >= 0 && rel_id % p.y_stride == 0) tgt_col = rel_id / p.y_stride;
      }
      int cnt = 0;
      float hi = tgt, lo = tgt;
      if constexpr (BAND) {
        const float mg = valid_x ? p.margin[x_global] : 0.f;
        hi = tgt + mg;
        lo = tgt - mg;
      }
      // scores at or below `floor_s` cannot be among the row's k best: some finished segment already holds k better
      float floor_s = -CUDART_INF_F;
      if constexpr (TOPK) {
        if (valid_x && p.row_floor != nullptr) floor_s = p.row_floor[x_global];
      }
      if constexpr (COLLECT) floor_s = valid_x ? p.row_floor[x_global] : CUDART_INF_F;
      float thr = valid_x ? floor_s : CUDART_INF_F;
      int minpos = 0;
      if constexpr (TOPK) {
        for (int j = 0; j < p.k; ++j) { top_s[j] = -CUDART_INF_F; top_i[j] = -1; }
      }

      for (int t = 0; t < n; ++t, ++g) {
        const uint32_t b = g % NBUF;
        if (!mbar_wait_bounded(s_full + b, (g / NBUF) & 1, s_abort)) { ok = false; break; }
        tc_fence_after();
        const int tile_col0 = (y0 + t) * BLOCK_Y;
        const int y_valid = p.y_rows - tile_col0;
        const uint32_t s_addr = tmem_base + b * BLOCK_Y + lane_sel;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int col0 = half * 64 + c * 32;
          uint32_t r[32];
          tmem_ld32(s_addr + col0, r);
          tc_wait_ld();
          const int rel = tgt_col - (tile_col0 + col0);  // position of the true entity inside this chunk, if any
          uint32_t band = 0u;
          const bool plain = (col0 + 32 <= y_valid) && (p.col_bias == nullptr);
          if (plain) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float s = __uint_as_float(r[i]);
              cnt += (s > hi && i != rel) ? 1 : 0;
              if constexpr (BAND) band |= ((s > lo && s <= hi && i != rel) ? 1u : 0u) << i;
              if constexpr (COLLECT) band |= (s >= floor_s ? 1u : 0u) << i;
              if constexpr (TOPK) {
                if (s > thr) {
                  top_s[minpos] = s;
                  top_i[minpos] = p.y_offset + (tile_col0 + col0 + i) * p.y_stride;
                  thr = top_s[0];
                  minpos = 0;
                  for (int j = 1; j < p.k; ++j)
                    if (top_s[j] < thr) { thr = top_s[j]; minpos = j; }
                  thr = fmaxf(thr, floor_s);
                }
              }
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const bool in = col0 + i < y_valid;
              float s = __uint_as_float(r[i]);
              if (p.col_bias != nullptr && in) s += p.col_bias[tile_col0 + col0 + i];
              if (!in) s = -CUDART_INF_F;
              cnt += (s > hi && i != rel) ? 1 : 0;
              if constexpr (BAND) band |= ((s > lo && s <= hi && i != rel) ? 1u : 0u) << i;
              if constexpr (COLLECT) band |= (s >= floor_s ? 1u : 0u) << i;
              if constexpr (TOPK) {
                if (s > thr) {
                  top_s[minpos] = s;
                  top_i[minpos] = p.y_offset + (tile_col0 + col0 + i) * p.y_stride;
                  thr = top_s[0];
                  minpos = 0;
                  for (int j = 1; j < p.k; ++j)
                    if (top_s[j] < thr) { thr = top_s[j]; minpos = j; }
                  thr = fmaxf(thr, floor_s);
                }
              }
            }
          }
          if constexpr (COLLECT) {
            while (band) {  // rare: the floor is the k-th best score of a sample of the table
              const int i = __ffs(band) - 1;
              band &= band - 1;
              const int pos = atomicAdd(p.cand_count + x_global, 1);
              if (pos < p.cand_cap) {
                float s = __uint_as_float(r[0]);
#pragma unroll
                for (int u = 1; u < 32; ++u) s = (u == i) ? __uint_as_float(r[u]) : s;
                if (p.col_bias != nullptr) s += p.col_bias[tile_col0 + col0 + i];
                p.cand_score[static_cast<size_t>(x_global) * p.cand_cap + pos] = s;
                p.cand_idx[static_cast<size_t>(x_global) * p.cand_cap + pos] =
                    p.y_offset + (tile_col0 + col0 + i) * p.y_stride;
              }
            }
          }
          if constexpr (BAND) {
            if (band != 0u) {  // undecided pairs of this thread's 32 columns go to the list of the exact pass
              const int nb = __popc(band);
              const unsigned long long base = atomicAdd(p.band_count, static_cast<unsigned long long>(nb));
              if (static_cast<long long>(base) + nb <= p.band_cap) {
                unsigned long long at = base;
                while (band) {
                  const int i = __ffs(band) - 1;
                  band &= band - 1;
                  p.band_rows[at] = x_global;
                  p.band_cols[at] = p.y_offset + (tile_col0 + col0 + i) * p.y_stride;
                  ++at;
                }
              } else {
                atomicCAS(p.status, 0, ST_INBOX_OVERFLOW);
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_empty + b);
      }
      if (!ok) break;
      if (valid_x) {
        if (p.greater != nullptr && cnt != 0) atomicAdd(p.greater + x_global, cnt);
        if constexpr (TOPK) {
          if (p.row_floor != nullptr && thr > floor_s) atomic_max_float(p.row_floor + x_global, thr);
          const int pos = atomicAdd(p.cand_count + x_global, p.k);
          if (pos + p.k <= p.cand_cap) {
            float* cs = p.cand_score + static_cast<size_t>(x_global) * p.cand_cap + pos;
            int* ci = p.cand_idx + static_cast<size_t>(x_global) * p.cand_cap + pos;
            for (int j = 0; j < p.k; ++j) { cs[j] = top_s[j]; ci[j] = top_i[j]; }
          } else {
            atomicCAS(p.status, 0, ST_INBOX_OVERFLOW);
          }
        }
      }
      w += n;
    }
    if (!ok) fail(ST_TIMEOUT_EPILOGUE);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int D, int MODE>
static int launch(const CUtensorMap& tx, const CUtensorMap& ty, const EvalParams& p, int num_ctas,
                  cudaStream_t stream) {
  auto kern = eval_rank_kernel<D, MODE>;
  static bool configured[64] = {false};   // the attribute is per device: one flag per device ordinal
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -3;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<D>::SMEM_BYTES) != cudaSuccess)
      return -3;
    configured[dev] = true;
  }
  kern<<<num_ctas, NUM_THREADS, Cfg<D>::SMEM_BYTES, stream>>>(tx, ty, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// One warp per query: dot products against gathered entity rows (bf16 operands, fp32 accumulation).
//   target_score[i]     = q_i · y[target[i]] (+ col_bias)
//   filtered_greater[i] = #{ j in filt_cols[filt_ptr[i] : filt_ptr[i+1]], j != target[i] : q_i · y_j (+ bias) > target_score[i] }
// Local row c of y is entity y_offset + c * y_stride; entities of other shards are skipped (the caller sums over
// shards).  With target_in != null the target scores are taken from it instead (second phase of the sharded
// protocol, after the owners' scores have been exchanged).
__device__ __forceinline__ float2 load2(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
__device__ __forceinline__ float2 load2(const float* p) { return *reinterpret_cast<const float2*>(p); }

template <typename T>
__global__ void eval_sparse_kernel(const T* __restrict__ q, const T* __restrict__ y, int n,
                                   int D, int y_rows, int y_offset, int y_stride, const int* __restrict__ target,
                                   const float* __restrict__ col_bias, const float* __restrict__ target_in,
                                   const long long* __restrict__ filt_ptr, const int* __restrict__ filt_cols,
                                   float* __restrict__ target_score, int* __restrict__ filtered_greater) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= n) return;
  const T* qi = q + static_cast<size_t>(warp) * D;
  auto dot = [&](int col) -> float {
    const T* yj = y + static_cast<size_t>(col) * D;
    float acc = 0.f;
    for (int d = lane * 2; d < D; d += 64) {
      const float2 a = load2(qi + d);
      const float2 b = load2(yj + d);
      acc = fmaf(a.x, b.x, acc);
      acc = fmaf(a.y, b.y, acc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (col_bias != nullptr) acc += col_bias[col];
    return acc;
  };
  auto local_row = [&](int e) -> int {
    const int r = e - y_offset;
    if (r < 0 || r % y_stride != 0) return -1;
    const int c = r / y_stride;
    return c < y_rows ? c : -1;
  };
  const int tg = target[warp];
  float ts;
  if (target_in != nullptr) {
    ts = target_in[warp];
  } else {
    const int tl = local_row(tg);
    if (tl < 0) return;  // not the owner: nothing to report in this phase
    ts = dot(tl);
    if (lane == 0 && target_score != nullptr) target_score[warp] = ts;
  }
  if (filt_ptr == nullptr || filtered_greater == nullptr) return;
  int cnt = 0;
  for (long long e = filt_ptr[warp]; e < filt_ptr[warp + 1]; ++e) {
    const int j = filt_cols[e];
    const int jl = local_row(j);
    if (j == tg || jl < 0) continue;
    cnt += dot(jl) > ts ? 1 : 0;
  }
  if (lane == 0) filtered_greater[warp] = cnt;
}

// Exact second pass of the band mode: one warp per undecided (query, entity) pair, fp32 operands; the pair counts
// when its exact score beats the exact target score of the query.
__global__ void eval_band_exact_kernel(const float* __restrict__ q, const float* __restrict__ y, int D, int y_rows,
                                       int y_offset, int y_stride, const float* __restrict__ col_bias,
                                       const int* __restrict__ band_rows, const int* __restrict__ band_cols,
                                       const unsigned long long* __restrict__ band_count, long long band_cap,
                                       const float* __restrict__ target, int* __restrict__ greater) {
  const long long total = min(static_cast<long long>(*band_count), band_cap);
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; i < total; i += warps) {
    const int row = band_rows[i];
    const int c = (band_cols[i] - y_offset) / y_stride;
    const float* qi = q + static_cast<size_t>(row) * D;
    const float* yj = y + static_cast<size_t>(c) * D;
    float acc = 0.f;
    for (int d = lane * 2; d < D; d += 64) {
      const float2 a = *reinterpret_cast<const float2*>(qi + d);
      const float2 b = *reinterpret_cast<const float2*>(yj + d);
      acc = fmaf(a.x, b.x, acc);
      acc = fmaf(a.y, b.y, acc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (col_bias != nullptr) acc += col_bias[c];
    if (lane == 0 && acc > target[row]) atomicAdd(greater + row, 1);
  }
}

}  // namespace evalk
}  // namespace dice

// Counts, for each query row, the columns of X · Yᵀ (+ col_bias) that exceed target[row], skipping the column
// target_idx[row]; with k > 0 also appends per-segment top-k candidates (k <= 32) to the row's candidate list,
// from which the caller takes the final top-k.  greater and cand_count must be zeroed, cand_score filled with -inf
// and cand_idx with -1 by the caller.  Row c of Y is entity y_offset + c * y_stride (sharded tables).
extern "C" int dice_eval_rank(const void* x, int x_rows, const void* y, int y_rows, int D, const float* target,
                              const int* target_idx, const float* col_bias, int y_offset, int y_stride, int* greater,
                              int k,
                              int cand_cap, float* cand_score, int* cand_idx, int* cand_count, int* status,
                              int num_ctas, const float* margin, int* band_rows, int* band_cols,
                              unsigned long long* band_count, long long band_cap, float* row_floor, void* stream) {
  using namespace dice;
  using namespace dice::evalk;
  if (x_rows <= 0 || y_rows <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(y) & 15)) return -5;
  if (k < -1 || k > KMAX) return -7;   // k == -1: collect mode (every score >= row_floor goes to the candidate lists)
  if (k != 0 && (cand_score == nullptr || cand_idx == nullptr || cand_count == nullptr || cand_cap < k)) return -7;
  if (k == -1 && row_floor == nullptr) return -7;
  CUtensorMap tx, ty;
  int rc = make_tmap_bf16(&tx, x, x_rows, D);
  if (rc) return rc;
  rc = make_tmap_bf16(&ty, y, y_rows, D);
  if (rc) return rc;
  EvalParams p;
  p.target = target;
  p.target_idx = target_idx;
  p.col_bias = col_bias;
  p.greater = greater;
  p.status = status;
  p.x_rows = x_rows;
  p.y_rows = y_rows;
  p.nx_tiles = (x_rows + BLOCK_X - 1) / BLOCK_X;
  p.ny_tiles = (y_rows + BLOCK_Y - 1) / BLOCK_Y;
  p.map = TileMap::make(p.nx_tiles, p.ny_tiles, BLOCK_Y * D * 2, 48ll << 20);
  p.y_offset = y_offset;
  p.y_stride = y_stride > 0 ? y_stride : 1;
  p.k = k;
  p.cand_cap = cand_cap;
  p.cand_score = cand_score;
  p.cand_idx = cand_idx;
  p.cand_count = cand_count;
  p.row_floor = row_floor;
  p.margin = margin;
  p.band_rows = band_rows;
  p.band_cols = band_cols;
  p.band_count = band_count;
  p.band_cap = band_cap;
  if (margin != nullptr && (k > 0 || band_rows == nullptr || band_cols == nullptr || band_count == nullptr)) return -7;
  if (num_ctas <= 0) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    num_ctas = sms;
  }
  const long long total = static_cast<long long>(p.nx_tiles) * p.ny_tiles;
  if (num_ctas > total) num_ctas = static_cast<int>(total);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int mode = k > 0 ? 1 : (k == -1 ? 3 : (margin != nullptr ? 2 : 0));
#define DICE_EVAL_DISPATCH(DD)                                              \
  case DD:                                                                  \
    if (mode == 1) return launch<DD, 1>(tx, ty, p, num_ctas, s);            \
    if (mode == 2) return launch<DD, 2>(tx, ty, p, num_ctas, s);            \
    if (mode == 3) return launch<DD, 3>(tx, ty, p, num_ctas, s);            \
    return launch<DD, 0>(tx, ty, p, num_ctas, s);
  switch (D) {
    DICE_EVAL_DISPATCH(256)
    DICE_EVAL_DISPATCH(128)
    DICE_EVAL_DISPATCH(64)
    default: return -6;
  }
}

// Number of candidate entries one row can receive from dice_eval_rank with the given shape: k per (segment, half),
// where the segments are found by walking every CTA's range in the kernel's own visiting order.
extern "C" int dice_eval_rank_cand_cap(int x_rows, int y_rows, int D, int k, int num_ctas) {
  using namespace dice;
  using namespace dice::evalk;
  if (num_ctas <= 0) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    num_ctas = sms;
  }
  const int nx = (x_rows + BLOCK_X - 1) / BLOCK_X, ny = (y_rows + BLOCK_Y - 1) / BLOCK_Y;
  const TileMap map = TileMap::make(nx, ny, BLOCK_Y * D * 2, 48ll << 20);
  const long long total = map.total();
  if (num_ctas > total) num_ctas = static_cast<int>(total);
  int* per_x = new int[nx]();
  for (int c = 0; c < num_ctas; ++c) {
    const long long w_end = total * (c + 1) / num_ctas;
    for (long long w = total * c / num_ctas; w < w_end;) {
      int x, y, run;
      map.locate(w, x, y, run);
      const long long n = run < w_end - w ? run : w_end - w;
      ++per_x[x];
      w += n;
    }
  }
  int worst = 1;
  for (int x = 0; x < nx; ++x) worst = per_x[x] > worst ? per_x[x] : worst;
  delete[] per_x;
  return worst * 2 * k;
}

extern "C" int dice_eval_sparse(const void* q, const void* y, int n, int D, int y_rows, int y_offset, int y_stride,
                                const int* target, const float* col_bias, const float* target_in,
                                const long long* filt_ptr, const int* filt_cols, float* target_score,
                                int* filtered_greater, int fp32_operands, void* stream) {
  using namespace dice::evalk;
  if (n <= 0) return 0;
  if (D % 2) return -6;
  const int threads = 256;
  const int blocks = (n * 32 + threads - 1) / threads;
  if (fp32_operands)
    eval_sparse_kernel<float><<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const float*>(q), static_cast<const float*>(y), n, D, y_rows, y_offset,
        y_stride > 0 ? y_stride : 1, target, col_bias, target_in, filt_ptr, filt_cols, target_score, filtered_greater);
  else
    eval_sparse_kernel<__nv_bfloat16><<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(y), n, D, y_rows, y_offset,
        y_stride > 0 ? y_stride : 1, target, col_bias, target_in, filt_ptr, filt_cols, target_score, filtered_greater);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Exact pass over the pairs that dice_eval_rank left undecided (band mode): q and y are the fp32 operands.
extern "C" int dice_eval_band_exact(const float* q, const float* y, int D, int y_rows, int y_offset, int y_stride,
                                    const float* col_bias, const int* band_rows, const int* band_cols,
                                    const unsigned long long* band_count, long long band_cap, const float* target,
                                    int* greater, void* stream) {
  using namespace dice::evalk;
  if (D % 2) return -6;
  eval_band_exact_kernel<<<148 * 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      q, y, D, y_rows, y_offset, y_stride > 0 ? y_stride : 1, col_bias, band_rows, band_cols, band_count, band_cap,
      target, greater);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
