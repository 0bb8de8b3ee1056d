// CTA-pair version of the fused KvsAll scoring + BCE + gradient kernel (sm_100a, tcgen05.mma.cta_group::2), D = 256.
//
// Same mathematics as kvsall_fused.cu (S = X·Yᵀ on the tensor cores, dS = sigmoid(S) − label formed in registers and
// fed back from TMEM, out += scale · dS · Y, optional loss), but two CTAs of a cluster work as ONE MMA unit on a
// 256-row X super-tile:
//
//   * each CTA keeps its own 128 rows of X in shared memory and its own 128 accumulator rows (out: 256 columns,
//     S: 2 x 128 columns) in its TMEM;
//   * of every 128-row Y tile a CTA loads only HALF per GEMM: rows [64 r, 64 r + 64) for S = X·Yᵀ (the pair MMA takes
//     N / 2 of the B operand from each CTA) and columns [128 r, 128 r + 128) for out += dS·Y.  Both halves are plain
//     per-CTA TMA loads of this GPU's memory; nothing is multicast.  Per unit of work a CTA therefore reads half
//     of the B operand from shared memory and receives half of the TMA traffic of the one-CTA kernel, whose first
//     GEMM is bound by exactly that bandwidth;
//   * the two halves live in separate rings (3 stages of 32 KB for the first GEMM, freed as soon as that GEMM has
//     read them; 2 stages of 32 KB for the second), so a Y stage is no longer held across the epilogue and the
//     tensor pipe does not wait for refills.
//
// The leader CTA (cluster rank 0) issues every MMA.  TMA completion bytes of both CTAs are credited to the leader's
// "full" barriers (cp.async.bulk.tensor ... .cta_group::2 with the barrier address mapped to rank 0); the epilogue
// warps of both CTAs arrive on the leader's "dS ready" barriers; the leader releases buffers in both CTAs with
// tcgen05.commit ... .multicast::cluster.  Every wait is bounded; on a time-out the kernel records a status code,
// lets its copies land, frees TMEM and returns.
//
// Reference math being replaced: the 4 `torch.mm` of ComplEx.forward_k_vs_all plus BCEWithLogitsLoss and their
// autograd backward (dicee/models/complex.py:254-264, dicee/models/base_model.py:138).
#include "dice_b200.h"
#include "ptx_sm100.cuh"
#include "tile_map.cuh"
#include "tma_host.cuh"

#include <stdio.h>

namespace dice {
namespace pair {

constexpr int D = 256;
constexpr int ROWS_CTA = 128;            // X rows per CTA; a super-tile has 2 x 128
constexpr int BLOCK_Y = 128;
constexpr int XSLAB = 128 * 128;         // 128 rows x 64 bf16
constexpr int RSLAB = 64 * 128;          // 64 rows x 64 bf16 (row half of a Y tile, one 64-column K slab)
constexpr int CSLAB = 128 * 128;         // 128 rows x 64 bf16 (column half of a Y tile: two such slabs)
constexpr int X_BYTES = 4 * XSLAB;       // 64 KB
constexpr int R_BYTES = 4 * RSLAB;       // 32 KB per stage
constexpr int C_BYTES = 2 * CSLAB;       // 32 KB per stage
constexpr int NR = 3, NC = 2;
constexpr int NUM_EPI_WARPS = 16;
constexpr int NUM_THREADS = 64 + 32 * NUM_EPI_WARPS;
constexpr int SMEM_BYTES = X_BYTES + NR * R_BYTES + NC * C_BYTES + 1024 /*align*/ + 512 /*barriers*/;

struct Params {
  float* out;           // [x_rows, D] fp32, accumulated with red.add
  double* loss;
  int* status;
  int x_rows, y_rows;
  int nx_tiles, ny_tiles;   // nx_tiles counts 256-row super-tiles
  TileMap map;
  float base, scale;
  const uint32_t* mask;
  int mask_stride;
  float pos_delta;
  int loss_share;       // -1: every tile adds its loss terms; 0 / 1: only tiles whose 256 x 256 block of the (x, y)
                        // plane has that parity do (the other launch of the step takes the rest)
  long long* trace;     // optional [64 tiles][8] clock64 stamps written by the leader CTA of pair 0, else null
};

__device__ __forceinline__ float ex2f(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float rcpf(float x) { float y; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float tanhf_fast(float x) { float y; asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }

// log1p(e) / e on [0, 1] (degree-5 minimax fit): keeps the logarithm off the special-function unit
__device__ __forceinline__ float log1p_over_e(float e) {
  float q = -0.02397957257926464f;
  q = fmaf(q, e, 0.10150004923343658f);
  q = fmaf(q, e, -0.2102936953306198f);
  q = fmaf(q, e, 0.3252951502799988f);
  q = fmaf(q, e, -0.49937260150909424f);
  q = fmaf(q, e, 0.9999918341636658f);
  return q;
}

template <bool LOSS, bool MASK, bool FULL>
__device__ __forceinline__ void epilogue_chunk(const uint32_t (&r)[32], uint32_t mword, float base, float label_pos,
                                               int y_valid, uint32_t (&packed)[16], float& loss) {
  constexpr float LOG2E = 1.4426950408889634f;
  if constexpr (!LOSS && !MASK) {
    // uniform label: sigmoid(s) - base = 0.5 tanh(s / 2) + (0.5 - base), three instructions per logit
    const float c0 = 0.5f - base;
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      float d0 = fmaf(tanhf_fast(0.5f * __uint_as_float(r[i])), 0.5f, c0);
      float d1 = fmaf(tanhf_fast(0.5f * __uint_as_float(r[i + 1])), 0.5f, c0);
      if (!FULL && i >= y_valid) d0 = 0.f;
      if (!FULL && i + 1 >= y_valid) d1 = 0.f;
      __nv_bfloat162 v = __floats2bfloat162_rn(d0, d1);
      packed[i >> 1] = *reinterpret_cast<uint32_t*>(&v);
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    float ds2[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const float s = __uint_as_float(r[i + u]);
      float label = base;
      if constexpr (MASK) label = ((mword >> (i + u)) & 1u) ? label_pos : base;
      float sig;
      if constexpr (LOSS) {
        const float e = ex2f(-fabsf(s) * LOG2E);
        const float inv = rcpf(1.f + e);
        sig = s >= 0.f ? inv : 1.f - inv;
        float l = fmaf(log1p_over_e(e), e, fmaxf(s, 0.f));
        l = fmaf(-label, s, l);
        if (!FULL && i + u >= y_valid) l = 0.f;
        loss += l;
      } else {
        sig = fmaf(tanhf_fast(0.5f * s), 0.5f, 0.5f);
      }
      float d = sig - label;
      if (!FULL && i + u >= y_valid) d = 0.f;
      ds2[u] = d;
    }
    __nv_bfloat162 v = __floats2bfloat162_rn(ds2[0], ds2[1]);
    packed[i >> 1] = *reinterpret_cast<uint32_t*>(&v);
  }
}

template <bool LOSS, bool MASK>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
kvsall_pair_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_yr,
                   const __grid_constant__ CUtensorMap tmap_yc, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sX = smem;
  uint8_t* sR = smem + X_BYTES;
  uint8_t* sC = sR + NR * R_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sC + NC * C_BYTES);
  uint64_t* x_full = bars + 0;       // leader: bytes of both CTAs' X tiles
  uint64_t* x_empty = bars + 1;      // both CTAs: the X tile may be overwritten
  uint64_t* dx_full = bars + 2;      // both CTAs: the out accumulator of the segment is complete
  uint64_t* dx_empty = bars + 3;     // leader: both CTAs' epilogue warps have drained it
  uint64_t* s_full = bars + 4;       // [2] both CTAs
  uint64_t* ds_full = bars + 6;      // [2] leader: 2 x NUM_EPI_WARPS arrivals
  uint64_t* r_full = bars + 8;       // [NR] leader
  uint64_t* r_empty = bars + 11;     // [NR] both
  uint64_t* c_full = bars + 14;      // [NC] leader
  uint64_t* c_empty = bars + 16;     // [NC] both
  uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(bars + 20);
  volatile int* s_abort = reinterpret_cast<volatile int*>(bars + 21);   // [0] abort flag, [1] always zero

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_cta_rank();          // 0 = leader
  const bool leader = cta == 0;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  const long long total = static_cast<long long>(p.nx_tiles) * p.ny_tiles;
  const long long w_begin = total * pair_id / num_pairs;
  const long long w_end = total * (pair_id + 1) / num_pairs;

  if (threadIdx.x == 0) {
    mbar_init(x_full, 1);
    mbar_init(x_empty, 1);
    mbar_init(dx_full, 1);
    mbar_init(dx_empty, 2 * NUM_EPI_WARPS);
    for (int i = 0; i < 2; ++i) {
      mbar_init(s_full + i, 1);
      mbar_init(ds_full + i, 2 * NUM_EPI_WARPS);
    }
    for (int i = 0; i < NR; ++i) { mbar_init(r_full + i, 1); mbar_init(r_empty + i, 1); }
    for (int i = 0; i < NC; ++i) { mbar_init(c_full + i, 1); mbar_init(c_empty + i, 1); }
    *reinterpret_cast<volatile uint64_t*>(bars + 21) = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_base_smem, 512);
    tmem_relinquish_pair();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_x);
    tma_prefetch_desc(&tmap_yr);
    tma_prefetch_desc(&tmap_yc);
  }
  tc_fence_before();
  cluster_sync_all();     // barriers of both CTAs are initialised before anything can signal them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_smem;
  const uint32_t tmem_out = tmem_base;
  const uint32_t tmem_s0 = tmem_base + 256;

  auto fail = [&](int code) {
    atomicCAS(p.status, 0, code);
    *s_abort = 1;
  };
  // pipeline diagnostics: 0 row-half load issued, 1 S GEMM issued, 2 second GEMM issued, 3 epilogue sees S,
  // 4 epilogue wrote dS, 5 out tile drained, 6 column-half load issued, 7 second GEMM found its inputs ready
  const bool tracing = p.trace != nullptr && blockIdx.x == 0;
  auto stamp = [&](uint32_t tile, int slot) {
    if (tracing && tile < 64) p.trace[tile * 8 + slot] = clock64();
  };

  if (warp == 0) {
    // =========================================================================== TMA producer (one per CTA)
    // Two independent load streams (row halves + X tiles for the first GEMM, column halves for the second) are
    // issued by one thread in whichever order their buffers become free: a stream never waits behind the other.
    if (lane == 0) {
      const uint32_t xf = map_to_cta(smem_u32(x_full), 0);
      // cursor of the row-half stream (X tile once per segment, then one row half per tile)
      long long wr = w_begin;
      int nr = 0, tr = 0, xr = 0, yr0 = 0;
      uint32_t rcount = 0, segr = 0;
      bool x_issued = false;
      // cursor of the column-half stream
      long long wc = w_begin;
      int nc = 0, tcur = 0, xc = 0, yc0 = 0;
      uint32_t ccount = 0;
      auto locate = [&](long long w, int& x, int& y0, int& n) {
        int run;
        p.map.locate(w, x, y0, run);
        n = static_cast<int>(min(static_cast<long long>(run), w_end - w));
      };
      if (wr < w_end) locate(wr, xr, yr0, nr);
      if (wc < w_end) locate(wc, xc, yc0, nc);
      uint32_t idle = 0;
      bool ok = true;
      while ((wr < w_end || wc < w_end) && ok && !*s_abort) {
        bool progressed = false;
        if (wr < w_end) {
          if (!x_issued && mbar_test_wait(x_empty, (segr & 1) ^ 1)) {
            if (leader) mbar_arrive_expect_tx(x_full, 2 * X_BYTES);
            const int x_row = xr * 2 * ROWS_CTA + static_cast<int>(cta) * ROWS_CTA;
            for (int s = 0; s < 4; ++s) tma_load_2d_pair(sX + s * XSLAB, &tmap_x, s * 64, x_row, xf);
            x_issued = true;
            progressed = true;
          }
          if (tr < nr && mbar_test_wait(r_empty + (rcount % NR), ((rcount / NR) & 1) ^ 1)) {
            const uint32_t rs = rcount % NR;
            stamp(rcount, 0);
            if (leader) mbar_arrive_expect_tx(r_full + rs, 2 * R_BYTES);
            const uint32_t rf = map_to_cta(smem_u32(r_full + rs), 0);
            uint8_t* rdst = sR + rs * R_BYTES;
            const int y_row = (yr0 + tr) * BLOCK_Y + static_cast<int>(cta) * 64;
            for (int s = 0; s < 4; ++s)   // rows [64 cta, 64 cta + 64) of the tile, all four K slabs
              tma_load_2d_pair(rdst + s * RSLAB, &tmap_yr, s * 64, y_row, rf);
            ++rcount;
            ++tr;
            progressed = true;
          }
          if (tr == nr && x_issued) {   // segment complete on the load side: move on
            wr += nr;
            ++segr;
            tr = 0;
            x_issued = false;
            if (wr < w_end) locate(wr, xr, yr0, nr);
          }
        }
        if (wc < w_end) {
          const uint32_t cs = ccount % NC;
          if (mbar_test_wait(c_empty + cs, ((ccount / NC) & 1) ^ 1)) {
            stamp(ccount, 6);
            if (leader) mbar_arrive_expect_tx(c_full + cs, 2 * C_BYTES);
            const uint32_t cf = map_to_cta(smem_u32(c_full + cs), 0);
            uint8_t* cdst = sC + cs * C_BYTES;
            const int y_row = (yc0 + tcur) * BLOCK_Y;
            for (int s = 0; s < 2; ++s)   // all 128 rows, columns [128 cta, 128 cta + 128)
              tma_load_2d_pair(cdst + s * CSLAB, &tmap_yc, static_cast<int>(cta) * 128 + s * 64, y_row, cf);
            ++ccount;
            progressed = true;
            if (++tcur == nc) { wc += nc; tcur = 0; if (wc < w_end) locate(wc, xc, yc0, nc); }
          }
        }
        if (progressed) {
          idle = 0;
        } else if (++idle > DICE_WAIT_LIMIT) {
          ok = false;
        } else if (idle > 64) {
          __nanosleep(32);
        }
      }
      if (!ok) fail(ST_TIMEOUT_PRODUCER);
      if (*s_abort) {
        // let the copies this thread issued land before the CTA may exit (their completion is credited to the
        // leader's barriers, which the other CTA cannot poll): a fixed pause far above any TMA latency
        for (int i = 0; i < 400; ++i) __nanosleep(250);
      }
    }
  } else if (warp == 1) {
    // =========================================================================== MMA issuer (leader CTA only)
    if (leader && lane == 0) {
      constexpr uint32_t IDESC_G1 = make_idesc_bf16(2 * ROWS_CTA, BLOCK_Y, 0, 0);   // S = X · Yᵀ, M = 256, N = 128
      constexpr uint32_t IDESC_G2 = make_idesc_bf16(2 * ROWS_CTA, D, 0, 1);         // out += dS · Y, N = 256, B MN-major
      const uint64_t xdesc = make_sw128_desc(smem_u32(sX), 16, 1024);
      const uint64_t rdesc = make_sw128_desc(smem_u32(sR), 16, 1024);
      const uint64_t cdesc = make_sw128_desc(smem_u32(sC), CSLAB, 1024);

      auto issue_g1 = [&](uint32_t gi) {
        const uint32_t rs = gi % NR;
        stamp(gi, 1);
        tc_fence_after();
        const uint64_t rd = rdesc + rs * (R_BYTES >> 4);
        const uint32_t d_tmem = tmem_s0 + (gi & 1) * BLOCK_Y;
#pragma unroll
        for (int sl = 0; sl < 4; ++sl) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint32_t a_off = sl * (XSLAB >> 4) + kk * 2;   // 16 bf16 = 32 bytes inside the swizzle span
            const uint32_t b_off = sl * (RSLAB >> 4) + kk * 2;
            mma_ss_pair(d_tmem, xdesc + a_off, rd + b_off, IDESC_G1, (sl | kk) ? 1u : 0u);
          }
        }
        tc_commit_pair(s_full + (gi & 1), 3);
        tc_commit_pair(r_empty + rs, 3);       // the row halves of this tile may be refilled in both CTAs
      };
      auto issue_g2 = [&](uint32_t gi, bool first, bool last) {
        const uint32_t cs = gi % NC;
        stamp(gi, 2);
        tc_fence_after();
        const uint64_t cd = cdesc + cs * (C_BYTES >> 4);
        const uint32_t a_base = tmem_s0 + (gi & 1) * BLOCK_Y;
#pragma unroll
        for (int k = 0; k < BLOCK_Y / 16; ++k) {
          const uint32_t a_tmem = a_base + 32 * (k >> 1) + 8 * (k & 1);
          mma_ts_pair(tmem_out, a_tmem, cd + k * 128, IDESC_G2, (k == 0 && first) ? 0u : 1u);
        }
        tc_commit_pair(c_empty + cs, 3);
        if (last) tc_commit_pair(dx_full, 3);
      };

      // cursors over this pair's range of (super-tile, y tile) numbers for the two GEMM streams
      long long w1 = w_begin, w2 = w_begin;
      int n1 = 0, n2 = 0, t1 = 0, t2 = 0;
      uint32_t seg1 = 0, seg2 = 0;
      auto load = [&](long long w, int& n) {
        int x, y0, run;
        p.map.locate(w, x, y0, run);
        n = static_cast<int>(min(static_cast<long long>(run), w_end - w));
      };
      if (w1 < w_end) { load(w1, n1); n2 = n1; }
      uint32_t g1 = 0, g2 = 0, idle = 0;
      bool ok = true;
      while (w2 < w_end && ok && !*s_abort) {
        bool progressed = false;
        if (g2 < g1 && mbar_test_wait(ds_full + (g2 & 1), (g2 >> 1) & 1) &&
            mbar_test_wait(c_full + (g2 % NC), (g2 / NC) & 1) &&
            (t2 != 0 || mbar_test_wait(dx_empty, (seg2 & 1) ^ 1))) {
          issue_g2(g2, t2 == 0, t2 + 1 == n2);
          ++g2;
          if (++t2 == n2) { w2 += n2; ++seg2; t2 = 0; if (w2 < w_end) load(w2, n2); }
          progressed = true;
        }
        if (!progressed && w1 < w_end && g1 - g2 < 2 && (t1 != 0 || mbar_test_wait(x_full, seg1 & 1)) &&
            mbar_test_wait(r_full + (g1 % NR), (g1 / NR) & 1)) {
          issue_g1(g1);
          if (t1 + 1 == n1) tc_commit_pair(x_empty, 3);   // last S GEMM of the segment: X may be refilled
          ++g1;
          if (++t1 == n1) { w1 += n1; ++seg1; t1 = 0; if (w1 < w_end) load(w1, n1); }
          progressed = true;
        }
        if (progressed) {
          idle = 0;
        } else if (++idle > DICE_WAIT_LIMIT) {
          ok = false;
        } else if (idle > 256) {
          __nanosleep(32);
        }
      }
      if (!ok) fail(ST_TIMEOUT_MMA);
    }
  } else {
    // =========================================================================== epilogue warps (both CTAs)
    const int quarter = warp & 3;
    const int cg = (warp - 2) >> 2;
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    const int row = quarter * 32 + lane;
    float loss_acc = 0.f;
    uint32_t g = 0, seg = 0;
    bool ok = true;
    const float label_pos = p.base + p.pos_delta;
    const uint32_t ds_remote0 = map_to_cta(smem_u32(ds_full), 0);
    const uint32_t dxe_remote = map_to_cta(smem_u32(dx_empty), 0);

    for (long long w = w_begin; w < w_end && ok && !*s_abort;) {
      int x, y0, run;
      p.map.locate(w, x, y0, run);
      const int n = static_cast<int>(min(static_cast<long long>(run), w_end - w));
      const int x_global = x * 2 * ROWS_CTA + static_cast<int>(cta) * ROWS_CTA + row;
      const bool valid_x = x_global < p.x_rows;
      float seg_loss = 0.f;
      const uint32_t* mrow = nullptr;
      uint32_t mnext = 0u;
      if constexpr (MASK) {
        if (valid_x) {
          mrow = p.mask + static_cast<size_t>(x_global) * p.mask_stride + y0 * 4 + cg;
          mnext = mrow[0];
        }
      }
      for (int t = 0; t < n; ++t, ++g) {
        const uint32_t b = g & 1;
        const uint32_t mword = mnext;
        if constexpr (MASK) {
          if (valid_x && t + 1 < n) mnext = mrow[(t + 1) * 4];
        }
        if (!mbar_wait_bounded(s_full + b, (g >> 1) & 1, s_abort)) { ok = false; break; }
        if (warp == 2 && lane == 0) stamp(g, 3);
        tc_fence_after();
        const int y_valid = p.y_rows - (y0 + t) * BLOCK_Y - cg * 32;
        const uint32_t s_addr = tmem_s0 + b * BLOCK_Y + lane_sel + cg * 32;
        uint32_t r[32];
        uint32_t packed[16];
        tmem_ld32(s_addr, r);
        tc_wait_ld();
        bool with_loss = LOSS;
        if constexpr (LOSS) with_loss = p.loss_share < 0 || ((x + ((y0 + t) >> 1)) & 1) == p.loss_share;
        if (with_loss) {
          if (y_valid >= 32) epilogue_chunk<LOSS, MASK, true>(r, mword, p.base, label_pos, y_valid, packed, seg_loss);
          else epilogue_chunk<LOSS, MASK, false>(r, mword, p.base, label_pos, y_valid, packed, seg_loss);
        } else {
          if (y_valid >= 32) epilogue_chunk<false, MASK, true>(r, mword, p.base, label_pos, y_valid, packed, seg_loss);
          else epilogue_chunk<false, MASK, false>(r, mword, p.base, label_pos, y_valid, packed, seg_loss);
        }
        tmem_st16(s_addr, packed);
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (warp == 2 && lane == 0) stamp(g, 4);
        if (lane == 0) mbar_arrive_cluster(ds_remote0 + b * 8);
      }
      if (!ok) break;
      if (valid_x) loss_acc += seg_loss;

      if (!mbar_wait_bounded(dx_full, seg & 1, s_abort)) { ok = false; break; }
      tc_fence_after();
      float* out_row = p.out + static_cast<size_t>(valid_x ? x_global : 0) * D;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int col0 = cg * 64 + c * 32;
        uint32_t r[32];
        tmem_ld32(tmem_out + lane_sel + col0, r);
        tc_wait_ld();
        if (valid_x) {
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            red_add_v4(out_row + col0 + i, __uint_as_float(r[i]) * p.scale, __uint_as_float(r[i + 1]) * p.scale,
                       __uint_as_float(r[i + 2]) * p.scale, __uint_as_float(r[i + 3]) * p.scale);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (warp == 2 && lane == 0) stamp(g - 1, 5);
      if (lane == 0) mbar_arrive_cluster(dxe_remote);
      w += n;
      ++seg;
    }
    if (!ok) fail(ST_TIMEOUT_EPILOGUE);
    if constexpr (LOSS) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) loss_acc += __shfl_xor_sync(0xffffffffu, loss_acc, o);
      if (lane == 0 && p.loss != nullptr) atomicAdd(p.loss, static_cast<double>(loss_acc));
    }
  }

  // =============================================================================== common tail
  __syncwarp();
  tc_fence_before();
  cluster_sync_all();     // neither CTA may leave (or free TMEM) while its partner can still signal or read it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

// [rows, 256] bf16 row-major, box = 64 columns x box_rows rows, 128-byte swizzle, out-of-range rows read as zero
static inline int make_tmap(CUtensorMap* m, const void* base, long long rows, int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return -1;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(D) * 2};
  cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}

template <bool LOSS, bool MASK>
static int launch(const CUtensorMap& tx, const CUtensorMap& tyr, const CUtensorMap& tyc, const Params& p,
                  int num_pairs, cudaStream_t stream) {
  auto kern = kvsall_pair_kernel<LOSS, MASK>;
  static bool configured[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -3;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return -3;
    configured[dev] = true;
  }
  kern<<<2 * num_pairs, NUM_THREADS, SMEM_BYTES, stream>>>(tx, tyr, tyc, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace pair
}  // namespace dice

// CTA-pair variant of dice_kvsall_fused for D = 256 (returns -6 for other widths: use dice_kvsall_fused there).
// num_pairs <= 0 selects one pair per two SMs.  loss_share (with_loss only): -1 = the loss of every (x, y) pair is
// added; 0 or 1 = only of the pairs whose 256 x 256 block has that parity, so that the two launches of a training
// step (roles of x and y swapped) can each take half of the loss arithmetic.  trace (optional, device int64 [64][8]): per-tile clock stamps of the
// leader CTA of pair 0 for pipeline diagnostics.
extern "C" int dice_kvsall_pair(const void* x, int x_rows, const void* y, int y_rows, int D, float* out, double* loss,
                                float base, float scale, int with_loss, int* status, int num_pairs,
                                const unsigned int* mask, int mask_stride, float pos_delta, int loss_share,
                                long long* trace, void* stream) {
  using namespace dice;
  using namespace dice::pair;
  if (x_rows <= 0 || y_rows <= 0) return 0;
  if (D != pair::D) return -6;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(y) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15))
    return -5;
  if (mask != nullptr && ((mask_stride & 3) || (reinterpret_cast<uintptr_t>(mask) & 7))) return -5;
  CUtensorMap tx, tyr, tyc;
  int rc = make_tmap(&tx, x, x_rows, 128);
  if (rc) return rc;
  rc = make_tmap(&tyr, y, y_rows, 64);
  if (rc) return rc;
  rc = make_tmap(&tyc, y, y_rows, 128);
  if (rc) return rc;
  Params p;
  p.out = out;
  p.loss = loss;
  p.status = status;
  p.x_rows = x_rows;
  p.y_rows = y_rows;
  p.nx_tiles = (x_rows + 2 * ROWS_CTA - 1) / (2 * ROWS_CTA);
  p.ny_tiles = (y_rows + BLOCK_Y - 1) / BLOCK_Y;
  p.map = TileMap::make(p.nx_tiles, p.ny_tiles, BLOCK_Y * pair::D * 2, 48ll << 20);
  p.base = base;
  p.scale = scale;
  p.mask = mask;
  p.mask_stride = mask_stride;
  p.pos_delta = pos_delta;
  p.trace = trace;
  p.loss_share = loss_share;
  if (num_pairs <= 0) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    num_pairs = sms / 2;
  }
  const long long total = static_cast<long long>(p.nx_tiles) * p.ny_tiles;
  if (num_pairs > total) num_pairs = static_cast<int>(total);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool wl = with_loss != 0, mk = mask != nullptr;
  if (wl) return mk ? launch<true, true>(tx, tyr, tyc, p, num_pairs, s) : launch<true, false>(tx, tyr, tyc, p, num_pairs, s);
  return mk ? launch<false, true>(tx, tyr, tyc, p, num_pairs, s) : launch<false, false>(tx, tyr, tyc, p, num_pairs, s);
}
