// Pieces of the tensor-core scoring kernel (kvsall_fused.cu) that do not depend on its tile sizes: launch parameters, the cursor over
// a CTA's range of tiles, and the epilogue arithmetic that turns logits into loss terms and dS.
#pragma once
#include "dice_b200.h"
#include "ptx_sm100.cuh"
#include "tile_map.cuh"

namespace dice {

struct KvsAllParams {
  float* out;           // [x_rows, D] fp32, accumulated with red.add
  double* loss;         // scalar accumulator (may be null when LOSS == false)
  int* status;          // 0 = ok, otherwise first failure code
  int x_rows, y_rows;   // valid row counts
  int nx_tiles, ny_tiles;
  TileMap map;          // visiting order of the (x tile, y tile) pairs
  float base;           // label value outside the positives (smoothing term)
  float scale;          // factor applied to out (1 / (B * |E|) for a mean-reduced loss)
  const uint32_t* mask; // MASK: bit y of row x set where (x, y) is a positive label; row stride mask_stride words
  int mask_stride;      // (a multiple of 4, so the two words a thread needs per tile are one aligned 8-byte load)
  float pos_delta;      // label(positive) - base
  long long* trace;     // optional [64 tiles][8] clock64 stamps written by CTA 0 (pipeline diagnostics), else null
  // SCORE != 0: the logit is a function of the dot product and one scalar per row of X and of Y
  const float* x_bias;  // [nx_tiles * 128] or null (= 0): SCORE 1 bias of row x; SCORE 2 squared norm of row x
  const float* y_bias;  // [ny_tiles * 128] or null (= 0), padded to whole tiles: the same for the rows of Y
  float* x_dsum;        // optional [x_rows]: += scale * sum over y of the value fed to the second GEMM
  float margin;         // SCORE 2: logit = margin - sqrt(|x|^2 + |y|^2 - 2 x.y)
  // Optimiser fused into the drain (opt.param != null): out is then the gradient buffer of the rows of X, and the CTA
  // whose partial sums complete an x tile (tile counters) updates those 128 rows at once: master weights, moments,
  // the bf16 rows that X itself is (no CTA reads a completed tile again) and clears the gradient.
  DiceFusedOptimizer opt;
};

__device__ __forceinline__ float fast_lg2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}


// Position of one GEMM stream inside this CTA's range of flattened (x tile, y tile) pairs; a segment is a run of
// tiles sharing the x tile.
struct TileCursor {
  long long w, w_end;
  TileMap map;
  int x, y0, t, n;
  uint32_t seg;
  __device__ __forceinline__ void load() {
    int run;
    map.locate(w, x, y0, run);
    n = static_cast<int>(min(static_cast<long long>(run), w_end - w));
  }
  __device__ __forceinline__ void start(long long wb, long long we, const TileMap& m) {
    w = wb; w_end = we; map = m; t = 0; seg = 0; x = 0; y0 = 0; n = 0;
    if (w < w_end) load();
  }
  __device__ __forceinline__ bool done() const { return w >= w_end; }
  __device__ __forceinline__ bool first() const { return t == 0; }
  __device__ __forceinline__ bool last() const { return t + 1 == n; }
  __device__ __forceinline__ void advance() {
    if (++t == n) {
      w += n;
      ++seg;
      t = 0;
      if (w < w_end) load();
    }
  }
};

// One thread's N logits of a tile (bit i of mword is the label of logit i): dS = sigmoid(s) - label packed as bf16 pairs (low half = even column) and, with
// LOSS, the BCE-with-logits terms added to lacc.  FULL: all N columns are valid entries of Y.
// SCORE selects how the logit follows from the dot product a = x.y of the tensor cores:
//   0  s = a
//   1  s = a + xb + yb[col]                     (per-query scalar terms of the Clifford models)
//   2  s = margin - sqrt(xb + yb[col] - 2 a)    (translational distance; xb, yb are squared norms).  The value handed
//      to the second GEMM is then dS / distance, and the caller subtracts (sum of those values) * x from the result:
//      d s / d x = (y - x) / distance.
// dsum accumulates the values handed to the second GEMM (SCORE != 0 only).
//
// The epilogue is bound by instruction issue (sixteen warps share four schedulers), so everything is derived from one
// hyperbolic tangent of the non-positive half argument, t = tanh(-|s| / 2) in (-1, 0]:
//   sigmoid(|s|) = u = 0.5 - 0.5 t  in [0.5, 1)        (no cancellation)
//   tanh(s / 2)  = t with its sign flipped where s >= 0 (one logic op on the sign bits)
//   dS = sigmoid(s) - label = 0.5 tanh(s / 2) + c      with c = 0.5 - label (one of two constants, picked by the mask)
//   BCE(s, label) = softplus(s) - label s = c s + 0.5 |s| - ln 2 * lg2(u)
// and the three sums  sum c s,  sum |s|,  sum lg2(u)  are kept apart (lacc[0..2]) and combined once per segment.  The
// last one is the logarithm of a product: the N <= 32 factors u of a chunk (each in [0.5, 1), so the product stays above
// 2^-32) are multiplied up and ONE logarithm is taken per chunk.  That leaves one special-function operation (the
// tanh) and about ten other instructions per logit; the special-function unit (16 results per clock and SM) would
// otherwise need as many cycles per tile as the two GEMMs do.
template <int N, bool LOSS, bool MASK, bool FULL, int SCORE>
__device__ __forceinline__ void epilogue_chunk(const uint32_t (&r)[N], uint32_t mword, float base, float label_pos,
                                               int y_valid, uint32_t (&packed)[N / 2], float (&lacc)[3], float xb,
                                               const float* __restrict__ yb, float margin, float& dsum) {
  const float c_base = 0.5f - base, c_pos = 0.5f - label_pos;
  float uprod = 1.f;
#pragma unroll
  for (int i = 0; i < N; i += 2) {
    float ds2[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      float s = __uint_as_float(r[i + u]);
      float gscale = 1.f;
      if constexpr (SCORE == 1) s += xb + yb[i + u];
      if constexpr (SCORE == 2) {
        const float d2 = fmaxf(fmaf(-2.f, s, xb + yb[i + u]), 1e-12f);
        gscale = rsqrtf(d2);
        s = fmaf(-d2, gscale, margin);
      }
      float c = c_base;
      if constexpr (MASK) c = ((mword >> (i + u)) & 1u) ? c_pos : c_base;
      const bool valid = FULL || (i + u < y_valid);
      float th;  // tanh(s / 2)
      if constexpr (LOSS) {
        const float tn = fast_tanh(-0.5f * fabsf(s));
        th = __uint_as_float(__float_as_uint(tn) ^ (~__float_as_uint(s) & 0x80000000u));
        const float us = fmaf(-0.5f, tn, 0.5f);   // sigmoid(|s|)
        if (valid) {
          lacc[0] = fmaf(c, s, lacc[0]);
          lacc[1] += fabsf(s);
          uprod *= us;
        }
      } else {
        th = fast_tanh(0.5f * s);
      }
      float d = fmaf(0.5f, th, c);
      if constexpr (SCORE == 2) d *= gscale;
      if (!valid) d = 0.f;
      if constexpr (SCORE != 0) dsum += d;
      ds2[u] = d;
    }
    __nv_bfloat162 v = __floats2bfloat162_rn(ds2[0], ds2[1]);  // .x (low 16 bits) = even K element
    packed[i >> 1] = *reinterpret_cast<uint32_t*>(&v);
  }
  if constexpr (LOSS) lacc[2] += fast_lg2(uprod);
}

}  // namespace dice
