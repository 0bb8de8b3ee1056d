// Fused KvsAll / 1vsAll scoring + BCE + gradient kernel for sm_100a (tcgen05 + TMEM + TMA).
//
// One launch computes, for an "X" matrix [x_rows, D] and a "Y" matrix [y_rows, D] (both bf16, row-major),
//
//     S   = X · Yᵀ                                    (tensor cores, fp32 accumulators in TMEM)
//     L  += Σ_{valid} softplus(S) − base · S          (optional; the label-independent part of BCE-with-logits)
//     dS  = sigmoid(S) − base                         (never written to memory: it goes TMEM → registers → TMEM)
//     out += scale · dS · Y                           (second GEMM, A operand read from TMEM; fp32 red.add to global)
//
// The [x_rows, y_rows] logit matrix is never materialised.  Calling it with X = entity shard, Y = queries gives
// the entity-table gradient and the loss; calling it with X = queries, Y = entity shard gives the query gradient.
// Positive labels enter in one of two ways: as a bit mask (one bit per (x, y) pair, built per batch from the CSR of
// known tails; the epilogue then uses the full label) or, for tables too large for a mask, through a separate sparse
// correction (see elementwise.cu), because BCE(s, y) = softplus(s) − y·s splits into a dense label-free term and a
// term over the known tails only.
//
// Structure of a CTA (576 threads, one CTA per SM, persistent over a contiguous range of (x-tile, y-tile) pairs):
//   warp 0       TMA producer: X tile once per segment, Y tiles through a ring of stages
//   warp 1       tcgen05.mma issuer (one elected lane); owns the TMEM allocation
//   warps 2..17  epilogue: tcgen05.ld S → sigmoid / loss → tcgen05.st dS (bf16, packed) → final drain of out
// TMEM columns: [0, D) out accumulator, [256, 384) and [384, 512) the double-buffered S tiles; dS overwrites
// columns of the S buffer it was computed from (the warp's own 32 columns, so no other warp's unread data is
// touched).  Sixteen epilogue warps (four per scheduler) keep the special-function unit busy: with eight the
// epilogue of the loss variant took 1.7x the time of the two GEMMs of a tile.
// Every mbarrier wait is bounded; on a time-out the kernel records a status code, drains its TMA copies, frees
// TMEM and returns.
#include "dice_b200.h"
#include "optim.cuh"
#include "ptx_sm100.cuh"
#include "tile_map.cuh"
#include "tma_host.cuh"
#include "kvsall_common.cuh"
#include "launch_pdl.cuh"

#include <stdio.h>

namespace dice {

constexpr int BLOCK_X = 128;
constexpr int BLOCK_Y = 128;
constexpr int SLAB_BYTES = 128 * 128;  // 128 rows x 64 bf16 (one 128-byte swizzle span per row)
constexpr int NUM_EPI_WARPS = 16;   // four per TMEM lane quarter, each owning 32 of a tile's 128 S columns
constexpr int NUM_THREADS = 64 + 32 * NUM_EPI_WARPS;

template <int D>
struct Cfg {
  static constexpr int NSLAB = D / 64;
  static constexpr int TILE_BYTES = NSLAB * SLAB_BYTES;
  static constexpr int NSTAGE = (D == 256) ? 2 : 4;
  static constexpr int SMEM_BYTES = TILE_BYTES * (1 + NSTAGE) + 1024 /*align*/ + 512 /*barriers*/;
};

template <int D, bool LOSS, bool MASK, int SCORE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
kvsall_fused_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_y,
                    const KvsAllParams p) {
  using C = Cfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sX = smem;
  uint8_t* sY = smem + C::TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::TILE_BYTES * (1 + C::NSTAGE));
  uint64_t* x_full = bars + 0;
  uint64_t* x_empty = bars + 1;
  uint64_t* dx_full = bars + 2;
  uint64_t* dx_empty = bars + 3;
  uint64_t* s_full = bars + 4;       // [2]
  uint64_t* ds_full = bars + 6;      // [2]
  uint64_t* y_empty = bars + 8;      // [NSTAGE]
  uint64_t* y_full = bars + 12;      // [NSTAGE][4]: one per 64-column slab, so the S GEMM starts on the first slab
  uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(bars + 28);
  volatile int* s_abort = reinterpret_cast<volatile int*>(bars + 29);
  volatile int* s_last = reinterpret_cast<volatile int*>(bars + 30);   // this CTA completed the x tile (fused optimiser)
  uint64_t* opt_issued = bars + 31;   // all epilogue warps have issued the reductions of a segment
  uint64_t* opt_decided = bars + 32;  // s_last of the segment is valid

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // contiguous range of flattened (x tile, y tile) pairs of this CTA
  const long long total = static_cast<long long>(p.nx_tiles) * p.ny_tiles;
  const long long w_begin = total * blockIdx.x / gridDim.x;
  const long long w_end = total * (blockIdx.x + 1) / gridDim.x;

  if (threadIdx.x == 0) {
    mbar_init(x_full, 1);
    mbar_init(x_empty, 1);
    mbar_init(dx_full, 1);
    mbar_init(dx_empty, NUM_EPI_WARPS);
    for (int i = 0; i < 2; ++i) {
      mbar_init(s_full + i, 1);
      mbar_init(ds_full + i, NUM_EPI_WARPS);
    }
    for (int i = 0; i < C::NSTAGE; ++i) {
      mbar_init(y_empty + i, 1);
      for (int sl = 0; sl < C::NSLAB; ++sl) mbar_init(y_full + i * 4 + sl, 1);
    }
    mbar_init(opt_issued, NUM_EPI_WARPS);
    mbar_init(opt_decided, 1);
    *reinterpret_cast<volatile uint64_t*>(bars + 29) = 0;  // abort flag and an always-zero word next to it
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
  // everything above (barriers, tensor-memory allocation, descriptor prefetch) may overlap the previous kernel's tail
  griddep_wait();
  griddep_launch();
  const uint32_t tmem_out = tmem_base;              // D columns
  const uint32_t tmem_s0 = tmem_base + 256;         // two S buffers of 128 columns

  auto fail = [&](int code) {
    atomicCAS(p.status, 0, code);
    *s_abort = 1;
  };
  const bool tracing = p.trace != nullptr && blockIdx.x == 0;
  auto stamp = [&](uint32_t tile, int slot) {
    if (tracing && tile < 64) p.trace[tile * 8 + slot] = clock64();
  };

  if (warp == 0) {
    // =========================================================================== TMA producer
    if (lane == 0) {
      uint32_t ycount = 0, seg = 0;
      uint32_t x_loads = 0;
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
          stamp(ycount, 0);
          uint8_t* dst = sY + st * C::TILE_BYTES;
          for (int s = 0; s < C::NSLAB; ++s) {
            mbar_arrive_expect_tx(y_full + st * 4 + s, SLAB_BYTES);
            tma_load_2d(dst + s * SLAB_BYTES, &tmap_y, s * 64, (y0 + t) * BLOCK_Y, y_full + st * 4 + s);
          }
        }
        if (!ok) { fail(ST_TIMEOUT_PRODUCER); break; }
        w += n;
        ++seg;
      }
      // Drain: every copy this thread issued must have landed before the CTA may exit.
      if (*s_abort) {
        bool drained = true;
        if (x_loads > 0) drained &= mbar_wait_bounded(x_full, (x_loads - 1) & 1, s_abort + 1 /*always 0*/, 1u << 20);
        for (uint32_t i = 0; i < C::NSTAGE && i < ycount; ++i) {
          const uint32_t last = ycount - 1 - i;  // the most recent use of each stage
          for (int sl = 0; sl < C::NSLAB; ++sl)
            drained &= mbar_wait_bounded(y_full + (last % C::NSTAGE) * 4 + sl, (last / C::NSTAGE) & 1, s_abort + 1,
                                         1u << 20);
        }
        if (!drained) atomicExch(p.status, ST_TIMEOUT_DRAIN);
      }
    }
  } else if (warp == 1) {
    // =========================================================================== MMA issuer
    // The two GEMMs of consecutive tiles are issued in whichever order their inputs become ready: the second GEMM
    // of tile g (needs dS from the epilogue) ahead of the first GEMM of tile g + 2 (needs the Y stage that the
    // former releases), so that the tensor pipe has work while that stage is being refilled.
    if (lane == 0) {
      constexpr uint32_t IDESC_G1 = make_idesc_bf16(BLOCK_X, BLOCK_Y, 0, 0);  // S = X · Yᵀ, both K-major
      constexpr uint32_t IDESC_G2 = make_idesc_bf16(BLOCK_X, D, 0, 1);        // out += dS · Y, Y read MN-major
      // descriptors are built once; per MMA only the 14-bit start-address field (16-byte units) is advanced
      const uint64_t xdesc = make_sw128_desc(smem_u32(sX), 16, 1024);
      const uint64_t ydesc_g1 = make_sw128_desc(smem_u32(sY), 16, 1024);
      const uint64_t ydesc_g2 = make_sw128_desc(smem_u32(sY), SLAB_BYTES, 1024);

      auto issue_g1 = [&](uint32_t gi) -> bool {
        const uint32_t st = gi % C::NSTAGE;
        const uint32_t par = (gi / C::NSTAGE) & 1;
        stamp(gi, 1);
        tc_fence_after();
        const uint64_t yd = ydesc_g1 + st * (C::TILE_BYTES >> 4);
        const uint32_t d_tmem = tmem_s0 + (gi & 1) * BLOCK_Y;
#pragma unroll
        for (int sl = 0; sl < C::NSLAB; ++sl) {
          if (sl > 0) {  // slab 0 was probed by the caller
            if (!mbar_wait_bounded(y_full + st * 4 + sl, par, s_abort)) return false;
            tc_fence_after();
          }
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint32_t off16 = sl * (SLAB_BYTES >> 4) + kk * 2;  // 16 bf16 = 32 bytes inside the swizzle span
            if (sl == 0 && kk == 0) mma_ss(d_tmem, xdesc + off16, yd + off16, IDESC_G1, 0u);
            else mma_ss(d_tmem, xdesc + off16, yd + off16, IDESC_G1, 1u);
          }
        }
        tc_commit(s_full + (gi & 1));
        return true;
      };
      auto issue_g2 = [&](uint32_t gi, bool first, bool last) {
        const uint32_t st = gi % C::NSTAGE;
        stamp(gi, 2);
        tc_fence_after();
        const uint64_t yd = ydesc_g2 + st * (C::TILE_BYTES >> 4);
        const uint32_t a_base = tmem_s0 + (gi & 1) * BLOCK_Y;
#pragma unroll
        for (int k = 0; k < BLOCK_Y / 16; ++k) {
          // dS: the 32 K elements of column group c are packed into columns [32 c, 32 c + 16) of the S buffer
          const uint32_t a_tmem = a_base + 32 * (k >> 1) + 8 * (k & 1);
          // Y tile as [K = 128 rows, N = D]: N blocks of 64 are one slab apart, groups of 8 K-rows 1024 B apart;
          // 16 K-rows = 2048 bytes
          if (k == 0) mma_ts(tmem_out, a_tmem, yd, IDESC_G2, first ? 0u : 1u);
          else mma_ts(tmem_out, a_tmem, yd + k * 128, IDESC_G2, 1u);
        }
        tc_commit(y_empty + st);
        if (last) tc_commit(dx_full);
      };

      TileCursor c1, c2;
      c1.start(w_begin, w_end, p.map);
      c2.start(w_begin, w_end, p.map);
      uint32_t g1 = 0, g2 = 0, idle = 0;
      bool ok = true;
      while (!c2.done() && ok && !*s_abort) {
        bool progressed = false;
        if (g2 < g1 && mbar_test_wait(ds_full + (g2 & 1), (g2 >> 1) & 1) &&
            (!c2.first() || mbar_test_wait(dx_empty, (c2.seg & 1) ^ 1))) {
          issue_g2(g2, c2.first(), c2.last());
          ++g2;
          c2.advance();
          progressed = true;
        }
        if (!progressed && !c1.done() && g1 - g2 < 2 && (!c1.first() || mbar_test_wait(x_full, c1.seg & 1)) &&
            mbar_test_wait(y_full + (g1 % C::NSTAGE) * 4, (g1 / C::NSTAGE) & 1)) {
          if (!issue_g1(g1)) { ok = false; break; }
          if (c1.last()) tc_commit(x_empty);  // last S GEMM of the segment: the X buffer may be refilled
          ++g1;
          c1.advance();
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
    // =========================================================================== epilogue warps
    const int quarter = warp & 3;              // TMEM lane group this warp may access
    const int cg = (warp - 2) >> 2;            // which 32 of the 128 S columns
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    const int row = quarter * 32 + lane;
    float loss_acc = 0.f;
    uint32_t g = 0, seg = 0;
    bool ok = true;
    const float label_pos = p.base + p.pos_delta;

    for (long long w = w_begin; w < w_end && ok && !*s_abort;) {
      int x, y0, run;
      p.map.locate(w, x, y0, run);
      const int n = static_cast<int>(min(static_cast<long long>(run), w_end - w));
      const int x_global = x * BLOCK_X + row;
      const bool valid_x = x_global < p.x_rows;
      float seg_l[3] = {0.f, 0.f, 0.f};   // sum c s, sum |s|, sum lg2(sigmoid(|s|)) of this thread's logits
      float seg_dsum = 0.f;
      float xb = 0.f;
      if constexpr (SCORE != 0) {
        if (valid_x && p.x_bias != nullptr) xb = p.x_bias[x_global];
      }

      // label words are fetched one tile ahead: the strided global load would otherwise sit on the critical path
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
        // the 32 per-column scalars of this chunk: the same addresses in every lane (a broadcast from L1), fetched
        // before the wait for S
        float yb[SCORE != 0 ? 32 : 1];
        if constexpr (SCORE != 0) {
          if (p.y_bias != nullptr) {
            const float4* src = reinterpret_cast<const float4*>(p.y_bias + static_cast<size_t>(y0 + t) * BLOCK_Y + cg * 32);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float4 v = __ldg(src + i);
              yb[4 * i] = v.x; yb[4 * i + 1] = v.y; yb[4 * i + 2] = v.z; yb[4 * i + 3] = v.w;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) yb[i] = 0.f;
          }
        }
        if (!mbar_wait_bounded(s_full + b, (g >> 1) & 1, s_abort)) { ok = false; break; }
        if (warp == 2 && lane == 0) stamp(g, 3);
        tc_fence_after();
        const int y_valid = p.y_rows - (y0 + t) * BLOCK_Y - cg * 32;  // columns >= y_valid of this chunk are padding
        const uint32_t s_addr = tmem_s0 + b * BLOCK_Y + lane_sel + cg * 32;
        uint32_t r[32];
        tmem_ld32(s_addr, r);
        tc_wait_ld();
        uint32_t packed[16];
        if (y_valid >= 32) {
          epilogue_chunk<32, LOSS, MASK, true, SCORE>(r, mword, p.base, label_pos, y_valid, packed, seg_l, xb, yb,
                                                  p.margin, seg_dsum);
        } else {
          epilogue_chunk<32, LOSS, MASK, false, SCORE>(r, mword, p.base, label_pos, y_valid, packed, seg_l, xb, yb,
                                                   p.margin, seg_dsum);
        }
        tmem_st16(s_addr, packed);
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (warp == 2 && lane == 0) stamp(g, 4);
        if (lane == 0) mbar_arrive(ds_full + b);
      }
      if (!ok) break;
      if (valid_x) loss_acc += fmaf(0.5f, seg_l[1], seg_l[0]) - 0.6931471805599453f * seg_l[2];
      if constexpr (SCORE != 0) {
        if (valid_x && p.x_dsum != nullptr) atomicAdd(p.x_dsum + x_global, seg_dsum * p.scale);
      }

      // drain the accumulated out tile of this segment: this warp owns D / 4 of its columns
      if (!mbar_wait_bounded(dx_full, seg & 1, s_abort)) { ok = false; break; }
      tc_fence_after();
      float* out_row = p.out;
      if (valid_x) out_row = p.out + static_cast<size_t>(x_global) * D;
      constexpr int DC = D / 4;
      if constexpr (DC >= 32) {
#pragma unroll
        for (int c = 0; c < DC / 32; ++c) {
          const int col0 = cg * DC + c * 32;
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
      } else {
        const int col0 = cg * DC;
        uint32_t r[16];
        tmem_ld16(tmem_out + lane_sel + col0, r);
        tc_wait_ld();
        if (valid_x) {
#pragma unroll
          for (int i = 0; i < 16; i += 4)
            red_add_v4(out_row + col0 + i, __uint_as_float(r[i]) * p.scale, __uint_as_float(r[i + 1]) * p.scale,
                       __uint_as_float(r[i + 2]) * p.scale, __uint_as_float(r[i + 3]) * p.scale);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (warp == 2 && lane == 0) stamp(g - 1, 5);
      if (lane == 0) mbar_arrive(dx_empty);
      if (p.opt.param != nullptr) {
        // the y tiles of this segment are counted once all sixteen warps' reductions are on their way to L2; whoever
        // brings the count of the x tile to ny_tiles holds the last partial sum and applies the update.  The hand-shake
        // between the warps uses mbarriers with bounded waits, like every other wait of this kernel.
        __threadfence();
        __syncwarp();
        if (lane == 0) mbar_arrive(opt_issued);
        if (warp == 2) {
          if (!mbar_wait_bounded(opt_issued, seg & 1, s_abort)) { ok = false; break; }
          if (lane == 0) {
            __threadfence();
            *s_last = (atomicAdd(p.opt.count + x, static_cast<unsigned>(n)) + n == static_cast<unsigned>(p.ny_tiles)) ? 1 : 0;
            mbar_arrive(opt_decided);
          }
        }
        if (!mbar_wait_bounded(opt_decided, seg & 1, s_abort)) { ok = false; break; }
        const bool is_last = *s_last != 0;
        if (is_last) {
          __threadfence();
          const int rows = min(BLOCK_X, p.x_rows - x * BLOCK_X);
          const size_t base4 = static_cast<size_t>(x) * BLOCK_X * (D / 4);
          float4* __restrict__ pw = reinterpret_cast<float4*>(p.opt.param) + base4;
          float4* __restrict__ pg = reinterpret_cast<float4*>(p.out) + base4;
          float4* __restrict__ pm = reinterpret_cast<float4*>(p.opt.m) + base4;
          float4* __restrict__ pv = reinterpret_cast<float4*>(p.opt.v) + base4;
          uint2* __restrict__ ps = reinterpret_cast<uint2*>(p.opt.shadow) + base4;
          const int kind = p.opt.kind;
          const OptStepConsts c = opt_step_consts(kind, *p.opt.step + 1, p.opt.beta1, p.opt.beta2);
          for (int i = threadIdx.x - 64; i < rows * (D / 4); i += 32 * NUM_EPI_WARPS) {
            float4 wv = pw[i];
            const float4 gv = __ldcg(pg + i);   // the sums were formed in L2 by other SMs' reductions
            float4 m = make_float4(0.f, 0.f, 0.f, 0.f), v = m;
            if (kind != 2) { m = pm[i]; v = pv[i]; }
            wv.x = opt_update(kind, wv.x, gv.x, m.x, v.x, p.opt.lr, p.opt.beta1, p.opt.beta2, p.opt.eps, p.opt.weight_decay, c.inv_bc1, c.inv_sqrt_bc2, c.clip, c.first_step);
            wv.y = opt_update(kind, wv.y, gv.y, m.y, v.y, p.opt.lr, p.opt.beta1, p.opt.beta2, p.opt.eps, p.opt.weight_decay, c.inv_bc1, c.inv_sqrt_bc2, c.clip, c.first_step);
            wv.z = opt_update(kind, wv.z, gv.z, m.z, v.z, p.opt.lr, p.opt.beta1, p.opt.beta2, p.opt.eps, p.opt.weight_decay, c.inv_bc1, c.inv_sqrt_bc2, c.clip, c.first_step);
            wv.w = opt_update(kind, wv.w, gv.w, m.w, v.w, p.opt.lr, p.opt.beta1, p.opt.beta2, p.opt.eps, p.opt.weight_decay, c.inv_bc1, c.inv_sqrt_bc2, c.clip, c.first_step);
            pw[i] = wv;
            pg[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (kind != 2) { pm[i] = m; pv[i] = v; }
            __nv_bfloat162 lo = __floats2bfloat162_rn(wv.x, wv.y), hi = __floats2bfloat162_rn(wv.z, wv.w);
            uint2 pk;
            pk.x = *reinterpret_cast<uint32_t*>(&lo);
            pk.y = *reinterpret_cast<uint32_t*>(&hi);
            ps[i] = pk;
          }
          if (threadIdx.x == 64) p.opt.count[x] = 0u;   // ready for the next launch
        }
      }
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
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------ host side
template <int D, bool LOSS, bool MASK, int SCORE>
static int launch(const CUtensorMap& tx, const CUtensorMap& ty, const KvsAllParams& p, int num_ctas,
                  cudaStream_t stream) {
  auto kern = kvsall_fused_kernel<D, LOSS, MASK, SCORE>;
  static bool configured[64] = {false};   // the attribute is per device: one flag per device ordinal
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -3;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<D>::SMEM_BYTES) != cudaSuccess)
      return -3;
    configured[dev] = true;
  }
  return launch_pdl(kern, dim3(num_ctas), dim3(NUM_THREADS), Cfg<D>::SMEM_BYTES, stream, tx, ty, p) == cudaSuccess ? 0 : -4;
}

}  // namespace dice

// x, y: bf16 row-major with 16-byte aligned base; D in {64, 128, 256}.  out must be zero-initialised (or hold a
// running sum) by the caller; *loss likewise.  num_ctas <= 0 selects one CTA per SM.  Returns 0 on a successful
// launch; device-side failures are reported through *status.  trace (optional, device int64 [64][8]): CTA 0 writes
// clock64 stamps per tile into it (0 Y-load issued, 1 S GEMM issued, 2 second GEMM issued, 3 epilogue sees S,
// 4 epilogue wrote dS, 5 out tile drained) for pipeline diagnostics.
// score_mode 0: logit = x.y.  1: logit = x.y + x_bias[x] + y_bias[y].  2: logit = margin - sqrt(x_bias[x] + y_bias[y]
// - 2 x.y) with the squared row norms as x_bias / y_bias; out then holds sum_y w y with w = dS / distance and the
// caller subtracts x_dsum[x] * x.  Modes 1 and 2 need a label mask; x_bias / y_bias (either may be null = zeros) must
// be readable up to the next multiple of 128 rows; x_dsum (optional, [x_rows], caller-zeroed) receives scale * the row
// sums of the values fed to the second GEMM (mode 1: the gradient of x_bias).
// opt (optional): the optimiser step of the rows of X fused into this launch, see DiceFusedOptimizer; `out` must then
// already hold every other contribution to the gradient of those rows, and opt->shadow must be x itself.
extern "C" int dice_kvsall_fused(const void* x, int x_rows, const void* y, int y_rows, int D, float* out,
                                 double* loss, float base, float scale, int with_loss, int* status, int num_ctas,
                                 const unsigned int* mask, int mask_stride, float pos_delta, long long* trace, int score_mode,
                                 const float* x_bias, const float* y_bias, float* x_dsum, float margin,
                                 const DiceFusedOptimizer* opt, void* stream) {
  using namespace dice;
  if (x_rows <= 0 || y_rows <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(y) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15))
    return -5;
  CUtensorMap tx, ty;
  int rc = make_tmap_bf16(&tx, x, x_rows, D);
  if (rc) return rc;
  rc = make_tmap_bf16(&ty, y, y_rows, D);
  if (rc) return rc;
  KvsAllParams p;
  p.out = out;
  p.loss = loss;
  p.status = status;
  p.x_rows = x_rows;
  p.y_rows = y_rows;
  p.nx_tiles = (x_rows + BLOCK_X - 1) / BLOCK_X;
  p.ny_tiles = (y_rows + BLOCK_Y - 1) / BLOCK_Y;
  p.map = TileMap::make(p.nx_tiles, p.ny_tiles, BLOCK_Y * D * 2, 48ll << 20);
  p.base = base;
  p.scale = scale;
  p.mask = mask;
  p.mask_stride = mask_stride;
  p.pos_delta = pos_delta;
  p.trace = trace;
  p.x_bias = x_bias;
  p.y_bias = y_bias;
  p.x_dsum = x_dsum;
  p.margin = margin;
  if (opt != nullptr && opt->param != nullptr) {
    // the update is written over the rows of X: masters, moments and gradient must line up with them, 16-byte aligned
    if (opt->m == nullptr || opt->v == nullptr || opt->shadow != x || opt->count == nullptr || opt->step == nullptr ||
        ((reinterpret_cast<uintptr_t>(opt->param) | reinterpret_cast<uintptr_t>(opt->m) |
          reinterpret_cast<uintptr_t>(opt->v)) & 15) || opt->kind < 0 || opt->kind > 3)
      return -5;
    p.opt = *opt;
  } else {
    p.opt = DiceFusedOptimizer{};
  }
  if (score_mode < 0 || score_mode > 2 || (score_mode != 0 && mask == nullptr)) return -6;
  if (reinterpret_cast<uintptr_t>(y_bias) & 15) return -5;
  if (mask != nullptr && ((mask_stride & 3) || (reinterpret_cast<uintptr_t>(mask) & 7))) return -5;
  if (num_ctas <= 0) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    num_ctas = sms;
  }
  const long long total = static_cast<long long>(p.nx_tiles) * p.ny_tiles;
  if (num_ctas > total) num_ctas = static_cast<int>(total);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool wl = with_loss != 0;
  const bool mk = mask != nullptr;
#define DICE_DISPATCH(DD)                                                                        \
  case DD:                                                                                       \
    if (score_mode == 1)                                                                         \
      return wl ? launch<DD, true, true, 1>(tx, ty, p, num_ctas, s) : launch<DD, false, true, 1>(tx, ty, p, num_ctas, s); \
    if (score_mode == 2)                                                                         \
      return wl ? launch<DD, true, true, 2>(tx, ty, p, num_ctas, s) : launch<DD, false, true, 2>(tx, ty, p, num_ctas, s); \
    if (wl) return mk ? launch<DD, true, true, 0>(tx, ty, p, num_ctas, s) : launch<DD, true, false, 0>(tx, ty, p, num_ctas, s); \
    return mk ? launch<DD, false, true, 0>(tx, ty, p, num_ctas, s) : launch<DD, false, false, 0>(tx, ty, p, num_ctas, s);
  switch (D) {
    DICE_DISPATCH(256)
    DICE_DISPATCH(128)
    DICE_DISPATCH(64)
    default: return -6;
  }
}
