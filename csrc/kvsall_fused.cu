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
// Structure of a CTA (320 threads, one CTA per SM, persistent over a contiguous range of (x-tile, y-tile) pairs):
//   warp 0      TMA producer: X tile once per segment, Y tiles through a ring of stages
//   warp 1      tcgen05.mma issuer (one elected lane); owns the TMEM allocation
//   warps 2..9  epilogue: tcgen05.ld S → sigmoid / loss → tcgen05.st dS (bf16, packed) → final drain of out
// TMEM columns: [0, D) out accumulator, [256, 384) and [384, 512) the double-buffered S tiles; dS overwrites
// columns of the S buffer it was computed from (its own half, so no other warp's unread data is touched).
// Every mbarrier wait is bounded; on a time-out the kernel records a status code, drains its TMA copies, frees
// TMEM and returns.
#include "ptx_sm100.cuh"
#include "tma_host.cuh"

#include <stdio.h>

namespace dice {

constexpr int BLOCK_X = 128;
constexpr int BLOCK_Y = 128;
constexpr int SLAB_BYTES = 128 * 128;  // 128 rows x 64 bf16 (one 128-byte swizzle span per row)
constexpr int NUM_THREADS = 320;
constexpr int NUM_EPI_WARPS = 8;

struct KvsAllParams {
  float* out;           // [x_rows, D] fp32, accumulated with red.add
  float* const* out_table;  // optional: row x goes to out_table[x / out_block_rows] + (x % out_block_rows) * D, so
  int out_block_rows;       // that blocks of rows can live on different GPUs (peer pointers): GEMM -> reduce-scatter
  double* loss;         // scalar accumulator (may be null when LOSS == false)
  int* status;          // 0 = ok, otherwise first failure code
  int x_rows, y_rows;   // valid row counts
  int nx_tiles, ny_tiles;
  float base;           // label value outside the positives (smoothing term)
  float scale;          // factor applied to out (1 / (B * |E|) for a mean-reduced loss)
  const uint32_t* mask; // MASK: bit y of row x set where (x, y) is a positive label; row stride mask_stride words
  int mask_stride;      // (a multiple of 4, so the two words a thread needs per tile are one aligned 8-byte load)
  float pos_delta;      // label(positive) - base
};

template <int D>
struct Cfg {
  static constexpr int NSLAB = D / 64;
  static constexpr int TILE_BYTES = NSLAB * SLAB_BYTES;
  static constexpr int NSTAGE = (D == 256) ? 2 : 4;
  static constexpr int SMEM_BYTES = TILE_BYTES * (1 + NSTAGE) + 1024 /*align*/ + 512 /*barriers*/;
};

__device__ __forceinline__ float fast_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_lg2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_rcp(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D, bool LOSS, bool MASK>
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
  uint64_t* y_full = bars + 8;       // [NSTAGE]
  uint64_t* y_empty = bars + 8 + 4;  // [NSTAGE]
  uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* s_abort = reinterpret_cast<volatile int*>(bars + 17);

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
      mbar_init(y_full + i, 1);
      mbar_init(y_empty + i, 1);
    }
    *reinterpret_cast<volatile uint64_t*>(bars + 17) = 0;  // abort flag and an always-zero word next to it
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
  const uint32_t tmem_out = tmem_base;              // D columns
  const uint32_t tmem_s0 = tmem_base + 256;         // two S buffers of 128 columns

  auto fail = [&](int code) {
    atomicCAS(p.status, 0, code);
    *s_abort = 1;
  };

  if (warp == 0) {
    // =========================================================================== TMA producer
    if (lane == 0) {
      uint32_t ycount = 0, seg = 0;
      uint32_t x_loads = 0;
      for (long long w = w_begin; w < w_end && !*s_abort;) {
        const int x = static_cast<int>(w / p.ny_tiles);
        const int y0 = static_cast<int>(w % p.ny_tiles);
        const int n = static_cast<int>(min(static_cast<long long>(p.ny_tiles - y0), w_end - w));
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
      // Drain: every copy this thread issued must have landed before the CTA may exit.
      if (*s_abort) {
        bool drained = true;
        if (x_loads > 0) drained &= mbar_wait_bounded(x_full, (x_loads - 1) & 1, s_abort + 1 /*always 0*/, 1u << 20);
        for (uint32_t i = 0; i < C::NSTAGE && i < ycount; ++i) {
          const uint32_t last = ycount - 1 - i;  // the most recent use of each stage
          drained &= mbar_wait_bounded(y_full + (last % C::NSTAGE), (last / C::NSTAGE) & 1, s_abort + 1, 1u << 20);
        }
        if (!drained) atomicExch(p.status, ST_TIMEOUT_DRAIN);
      }
    }
  } else if (warp == 1) {
    // =========================================================================== MMA issuer
    if (lane == 0) {
      constexpr uint32_t IDESC_G1 = make_idesc_bf16(BLOCK_X, BLOCK_Y, 0, 0);  // S = X · Yᵀ, both K-major
      constexpr uint32_t IDESC_G2 = make_idesc_bf16(BLOCK_X, D, 0, 1);        // out += dS · Y, Y read MN-major
      const uint32_t sx_addr = smem_u32(sX);
      uint32_t g = 0, seg = 0;
      bool ok = true;

      auto issue_g1 = [&](uint32_t gi) -> bool {
        const uint32_t st = gi % C::NSTAGE;
        if (!mbar_wait_bounded(y_full + st, (gi / C::NSTAGE) & 1, s_abort)) return false;
        tc_fence_after();
        const uint32_t sy_addr = smem_u32(sY + st * C::TILE_BYTES);
        const uint32_t d_tmem = tmem_s0 + (gi & 1) * BLOCK_Y;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * SLAB_BYTES + (k & 3) * 32;  // 16 bf16 = 32 bytes inside the swizzle span
          mma_ss(d_tmem, make_sw128_desc(sx_addr + off, 16, 1024), make_sw128_desc(sy_addr + off, 16, 1024),
                 IDESC_G1, k > 0 ? 1u : 0u);
        }
        tc_commit(s_full + (gi & 1));
        return true;
      };
      auto issue_g2 = [&](uint32_t gi, bool first, bool last) -> bool {
        const uint32_t st = gi % C::NSTAGE;
        const uint32_t b = gi & 1;
        if (!mbar_wait_bounded(ds_full + b, (gi >> 1) & 1, s_abort)) return false;
        if (first && !mbar_wait_bounded(dx_empty, (seg & 1) ^ 1, s_abort)) return false;
        tc_fence_after();
        const uint32_t sy_addr = smem_u32(sY + st * C::TILE_BYTES);
        const uint32_t a_base = tmem_s0 + b * BLOCK_Y;
#pragma unroll
        for (int k = 0; k < BLOCK_Y / 16; ++k) {
          // dS columns: K elements 0..63 live in columns [0, 32), 64..127 in columns [64, 96) of the S buffer
          const uint32_t a_tmem = a_base + (k < 4 ? 8 * k : 64 + 8 * (k - 4));
          // Y tile as [K = 128 rows, N = D]: N blocks of 64 are one slab apart, groups of 8 K-rows 1024 B apart
          mma_ts(tmem_out, a_tmem, make_sw128_desc(sy_addr + k * 16 * 128, SLAB_BYTES, 1024), IDESC_G2,
                 (first && k == 0) ? 0u : 1u);
        }
        tc_commit(y_empty + st);
        if (last) tc_commit(dx_full);
        return true;
      };

      for (long long w = w_begin; w < w_end && ok && !*s_abort;) {
        const int y0 = static_cast<int>(w % p.ny_tiles);
        const int n = static_cast<int>(min(static_cast<long long>(p.ny_tiles - y0), w_end - w));
        if (!mbar_wait_bounded(x_full, seg & 1, s_abort)) { ok = false; break; }
        tc_fence_after();
        ok = issue_g1(g);
        if (ok && n == 1) tc_commit(x_empty);
        for (int t = 0; t < n && ok; ++t) {
          if (t + 1 < n) {
            ok = issue_g1(g + t + 1);
            if (ok && t + 2 == n) tc_commit(x_empty);  // last S GEMM of the segment: X buffer may be refilled
          }
          if (ok) ok = issue_g2(g + t, t == 0, t + 1 == n);
        }
        g += n;
        w += n;
        ++seg;
      }
      if (!ok) fail(ST_TIMEOUT_MMA);
    }
  } else {
    // =========================================================================== epilogue warps
    const int quarter = warp & 3;              // TMEM lane group this warp may access
    const int half = (warp - 2) >> 2;          // which 64 of the 128 S columns
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    const int row = quarter * 32 + lane;
    float loss_acc = 0.f;
    uint32_t g = 0, seg = 0;
    bool ok = true;
    constexpr float LOG2E = 1.4426950408889634f;
    constexpr float LN2 = 0.6931471805599453f;

    for (long long w = w_begin; w < w_end && ok && !*s_abort;) {
      const int x = static_cast<int>(w / p.ny_tiles);
      const int y0 = static_cast<int>(w % p.ny_tiles);
      const int n = static_cast<int>(min(static_cast<long long>(p.ny_tiles - y0), w_end - w));
      const int x_global = x * BLOCK_X + row;
      const bool valid_x = x_global < p.x_rows;
      float seg_loss = 0.f;

      for (int t = 0; t < n; ++t, ++g) {
        const uint32_t b = g & 1;
        uint2 mw = make_uint2(0u, 0u);
        if constexpr (MASK) {
          if (valid_x)
            mw = *reinterpret_cast<const uint2*>(p.mask + static_cast<size_t>(x_global) * p.mask_stride +
                                                 (y0 + t) * 4 + half * 2);
        }
        if (!mbar_wait_bounded(s_full + b, (g >> 1) & 1, s_abort)) { ok = false; break; }
        tc_fence_after();
        const int y_valid = p.y_rows - (y0 + t) * BLOCK_Y;  // columns >= y_valid are padding
        const uint32_t s_addr = tmem_s0 + b * BLOCK_Y + lane_sel;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int col0 = half * 64 + c * 32;
          uint32_t r[32];
          tmem_ld32(s_addr + col0, r);
          tc_wait_ld();
          uint32_t packed[16];
          const uint32_t mword = c == 0 ? mw.x : mw.y;
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float ds2[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const float s = __uint_as_float(r[i + u]);
              float label = p.base;
              if constexpr (MASK) label = ((mword >> (i + u)) & 1u) ? p.base + p.pos_delta : p.base;
              float sig;
              if constexpr (LOSS) {
                const float e = fast_ex2(-fabsf(s) * LOG2E);       // exp(-|s|)
                const float inv = fast_rcp(1.f + e);               // sigmoid(|s|)
                sig = s >= 0.f ? inv : e * inv;
                float l = fmaxf(s, 0.f) + LN2 * fast_lg2(1.f + e) - label * s;
                if (col0 + i + u >= y_valid) l = 0.f;
                seg_loss += l;
              } else {
                sig = fmaf(fast_tanh(0.5f * s), 0.5f, 0.5f);
              }
              float d = sig - label;
              if (col0 + i + u >= y_valid) d = 0.f;
              ds2[u] = d;
            }
            __nv_bfloat162 v = __floats2bfloat162_rn(ds2[0], ds2[1]);  // .x (low 16 bits) = even K element
            packed[i >> 1] = *reinterpret_cast<uint32_t*>(&v);
          }
          tmem_st16(s_addr + half * 64 + c * 16, packed);
        }
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(ds_full + b);
      }
      if (!ok) break;
      if (valid_x) loss_acc += seg_loss;

      // drain the accumulated out tile of this segment
      if (!mbar_wait_bounded(dx_full, seg & 1, s_abort)) { ok = false; break; }
      tc_fence_after();
      float* out_row = p.out;
      if (valid_x) {
        out_row = (p.out_table != nullptr)
                      ? p.out_table[x_global / p.out_block_rows] + static_cast<size_t>(x_global % p.out_block_rows) * D
                      : p.out + static_cast<size_t>(x_global) * D;
      }
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        const int col0 = half * (D / 2) + c * 32;
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
      if (lane == 0) mbar_arrive(dx_empty);
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
template <int D, bool LOSS, bool MASK>
static int launch(const CUtensorMap& tx, const CUtensorMap& ty, const KvsAllParams& p, int num_ctas,
                  cudaStream_t stream) {
  auto kern = kvsall_fused_kernel<D, LOSS, MASK>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<D>::SMEM_BYTES) != cudaSuccess)
      return -3;
    configured = true;
  }
  kern<<<num_ctas, NUM_THREADS, Cfg<D>::SMEM_BYTES, stream>>>(tx, ty, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace dice

// x, y: bf16 row-major with 16-byte aligned base; D in {64, 128, 256}.  out must be zero-initialised (or hold a
// running sum) by the caller; *loss likewise.  With out_table != null (a device array of base pointers, one per
// block of out_block_rows rows, possibly in peer memory) the result rows are scattered to their owners instead.  num_ctas <= 0 selects one CTA per SM.  Returns 0 on a successful
// launch; device-side failures are reported through *status.
extern "C" int dice_kvsall_fused(const void* x, int x_rows, const void* y, int y_rows, int D, float* out,
                                 double* loss, float base, float scale, int with_loss, int* status, int num_ctas,
                                 float* const* out_table, int out_block_rows, const unsigned int* mask,
                                 int mask_stride, float pos_delta, void* stream) {
  using namespace dice;
  if (x_rows <= 0 || y_rows <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(y) & 15) ||
      (out_table == nullptr && (reinterpret_cast<uintptr_t>(out) & 15)))
    return -5;
  CUtensorMap tx, ty;
  int rc = make_tmap_bf16(&tx, x, x_rows, D);
  if (rc) return rc;
  rc = make_tmap_bf16(&ty, y, y_rows, D);
  if (rc) return rc;
  KvsAllParams p;
  p.out = out;
  p.out_table = out_table;
  p.out_block_rows = out_block_rows > 0 ? out_block_rows : 1;
  p.loss = loss;
  p.status = status;
  p.x_rows = x_rows;
  p.y_rows = y_rows;
  p.nx_tiles = (x_rows + BLOCK_X - 1) / BLOCK_X;
  p.ny_tiles = (y_rows + BLOCK_Y - 1) / BLOCK_Y;
  p.base = base;
  p.scale = scale;
  p.mask = mask;
  p.mask_stride = mask_stride;
  p.pos_delta = pos_delta;
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
    if (wl) return mk ? launch<DD, true, true>(tx, ty, p, num_ctas, s) : launch<DD, true, false>(tx, ty, p, num_ctas, s); \
    return mk ? launch<DD, false, true>(tx, ty, p, num_ctas, s) : launch<DD, false, false>(tx, ty, p, num_ctas, s);
  switch (D) {
    DICE_DISPATCH(256)
    DICE_DISPATCH(128)
    DICE_DISPATCH(64)
    default: return -6;
  }
}
