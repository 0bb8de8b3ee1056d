// Convolutional gate of the ConEx / ConvQ / ConvO families: 1 -> C channel 3x3 convolution (padding 1) over the
// [2k, d/k] image made of the head's and the relation's blocks, batch normalisation (batch statistics when training,
// running statistics otherwise) and ReLU, forward and backward, without materialising the convolution output or its
// normalised copy.  The image of one sample is the 2d contiguous floats [head row | relation row].
//
// Forward, training:  conv_gate_stats (per-channel sum and sum of squares of the convolution output)
//                     conv_gate_finalize (mean, 1/std, folded scale and shift, running statistics)
//                     conv_gate_apply (recompute the convolution, normalise, ReLU, write the feature map)
// Forward, inference: conv_gate_finalize (from the running statistics) + conv_gate_apply
// Backward:           conv_gate_bwd_stats (d gamma, d beta), conv_gate_bwd_apply (d image, d weights, d bias)
//
// The reference runs the same chain as torch.cat -> nn.Conv2d -> nn.BatchNorm2d -> relu
// (dicee/models/complex.py:47-66, dicee/models/quaternion.py:262-283, dicee/models/octonion.py:214-236).
#include <cuda_runtime.h>
#include <stdint.h>

#include "dice_b200.h"

namespace {

constexpr int kThreads = 256;

struct GateShape {
  int B, H, W, C;   // samples, image rows (2k), image columns (d/k), output channels
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Copy one sample's image into a zero-bordered plane of (H+2) x (W+2) floats.
__device__ __forceinline__ void stage_image(const float* __restrict__ x, float* xs, int H, int W) {
  const int PW = W + 2, plane = (H + 2) * PW;
  for (int i = threadIdx.x; i < plane; i += blockDim.x) {
    int y = i / PW - 1, c = i % PW - 1;
    xs[i] = (y >= 0 && y < H && c >= 0 && c < W) ? x[y * W + c] : 0.f;
  }
}

__device__ __forceinline__ void load_patch(const float* xs, int y, int x, int PW, float (&nb)[9]) {
  const float* p = xs + y * PW + x;   // top-left of the 3x3 window in bordered coordinates
#pragma unroll
  for (int i = 0; i < 3; ++i)
#pragma unroll
    for (int j = 0; j < 3; ++j) nb[i * 3 + j] = p[i * PW + j];
}

__device__ __forceinline__ float conv_at(const float (&nb)[9], const float* w, float bias) {
  float z = bias;
#pragma unroll
  for (int t = 0; t < 9; ++t) z = fmaf(w[t], nb[t], z);
  return z;
}

// Block-level add of per-thread channel accumulators into double totals.
template <int CT>
__device__ __forceinline__ void reduce_to_global(float (&a)[CT], float (&b)[CT], int C, double* out_a, double* out_b,
                                                 float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
  for (int c = 0; c < CT; ++c) {
    if (c >= C) break;
    float sa = warp_sum(a[c]), sb = warp_sum(b[c]);
    if (lane == 0) { red[warp * 2] = sa; red[warp * 2 + 1] = sb; }
    __syncthreads();
    if (threadIdx.x == 0) {
      double ta = 0, tb = 0;
      for (int k = 0; k < nw; ++k) { ta += red[k * 2]; tb += red[k * 2 + 1]; }
      atomicAdd(out_a + c, ta);
      atomicAdd(out_b + c, tb);
    }
    __syncthreads();
  }
}

// stats[0..C) += sum z, stats[C..2C) += sum z^2
template <int CT>
__global__ void __launch_bounds__(kThreads) conv_gate_stats(GateShape s, const float* __restrict__ X,
                                                            const float* __restrict__ w, const float* __restrict__ bias,
                                                            double* __restrict__ stats) {
  extern __shared__ float sm[];
  float* ws = sm;                  // C*9
  float* bs = ws + CT * 9;         // C
  float* red = bs + CT;            // 2 * warps
  float* xs = red + 2 * (kThreads / 32);
  for (int i = threadIdx.x; i < s.C * 9; i += blockDim.x) ws[i] = w[i];
  for (int i = threadIdx.x; i < s.C; i += blockDim.x) bs[i] = bias[i];
  float a[CT], b[CT];
#pragma unroll
  for (int c = 0; c < CT; ++c) a[c] = b[c] = 0.f;
  const int HW = s.H * s.W, PW = s.W + 2;
  for (int n = blockIdx.x; n < s.B; n += gridDim.x) {
    __syncthreads();
    stage_image(X + (size_t)n * HW, xs, s.H, s.W);
    __syncthreads();
    for (int p = threadIdx.x; p < HW; p += blockDim.x) {
      float nb[9];
      load_patch(xs, p / s.W, p % s.W, PW, nb);
#pragma unroll
      for (int c = 0; c < CT; ++c) {
        if (c >= s.C) break;
        float z = conv_at(nb, ws + c * 9, bs[c]);
        a[c] += z;
        b[c] = fmaf(z, z, b[c]);
      }
    }
  }
  __syncthreads();
  reduce_to_global<CT>(a, b, s.C, stats, stats + s.C, red);
}

// One thread per channel.  training: batch statistics from `stats`, running statistics updated with `momentum`
// (unbiased variance, as torch.nn.BatchNorm2d does).  Otherwise the running statistics are used.
// fold[0..C) = gamma / std, fold[C..2C) = beta - mean * gamma / std, fold[2C..3C) = mean, fold[3C..4C) = 1 / std.
__global__ void conv_gate_finalize(int C, double count, int training, const double* __restrict__ stats,
                                   const float* __restrict__ gamma, const float* __restrict__ beta,
                                   float* __restrict__ run_mean, float* __restrict__ run_var, float momentum, float eps,
                                   float* __restrict__ fold) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float mean, var;
  if (training) {
    double m = stats[c] / count;
    double v = stats[C + c] / count - m * m;
    if (v < 0) v = 0;
    mean = (float)m;
    var = (float)v;
    if (run_mean != nullptr) {
      double unbiased = count > 1 ? v * count / (count - 1) : v;
      run_mean[c] = (1.f - momentum) * run_mean[c] + momentum * mean;
      run_var[c] = (1.f - momentum) * run_var[c] + momentum * (float)unbiased;
    }
  } else {
    mean = run_mean[c];
    var = run_var[c];
  }
  float inv = rsqrtf(var + eps);
  float g = gamma ? gamma[c] : 1.f, bt = beta ? beta[c] : 0.f;
  fold[c] = g * inv;
  fold[C + c] = bt - mean * g * inv;
  fold[2 * C + c] = mean;
  fold[3 * C + c] = inv;
}

// F[n, c, y, x] = relu(conv(n, c, y, x) * scale[c] + shift[c])
template <int CT>
__global__ void __launch_bounds__(kThreads) conv_gate_apply(GateShape s, const float* __restrict__ X,
                                                            const float* __restrict__ w, const float* __restrict__ bias,
                                                            const float* __restrict__ fold, float* __restrict__ F) {
  extern __shared__ float sm[];
  float* ws = sm;
  float* bs = ws + CT * 9;
  float* sc = bs + CT;
  float* sh = sc + CT;
  float* xs = sh + CT;
  for (int i = threadIdx.x; i < s.C * 9; i += blockDim.x) ws[i] = w[i];
  for (int i = threadIdx.x; i < s.C; i += blockDim.x) {
    bs[i] = bias[i];
    sc[i] = fold[i];
    sh[i] = fold[s.C + i];
  }
  const int HW = s.H * s.W, PW = s.W + 2;
  for (int n = blockIdx.x; n < s.B; n += gridDim.x) {
    __syncthreads();
    stage_image(X + (size_t)n * HW, xs, s.H, s.W);
    __syncthreads();
    float* out = F + (size_t)n * s.C * HW;
    for (int p = threadIdx.x; p < HW; p += blockDim.x) {
      float nb[9];
      load_patch(xs, p / s.W, p % s.W, PW, nb);
#pragma unroll
      for (int c = 0; c < CT; ++c) {
        if (c >= s.C) break;
        float y = fmaf(conv_at(nb, ws + c * 9, bs[c]), sc[c], sh[c]);
        out[(size_t)c * HW + p] = fmaxf(y, 0.f);
      }
    }
  }
}

// bstats[0..C) += sum dy * zhat (d gamma), bstats[C..2C) += sum dy (d beta), dy = dF where the ReLU was open.
template <int CT>
__global__ void __launch_bounds__(kThreads) conv_gate_bwd_stats(GateShape s, const float* __restrict__ X,
                                                                const float* __restrict__ w,
                                                                const float* __restrict__ bias,
                                                                const float* __restrict__ fold,
                                                                const float* __restrict__ dF,
                                                                double* __restrict__ bstats) {
  extern __shared__ float sm[];
  float* ws = sm;
  float* bs = ws + CT * 9;
  float* sc = bs + CT;
  float* sh = sc + CT;
  float* mu = sh + CT;
  float* iv = mu + CT;
  float* red = iv + CT;
  float* xs = red + 2 * (kThreads / 32);
  for (int i = threadIdx.x; i < s.C * 9; i += blockDim.x) ws[i] = w[i];
  for (int i = threadIdx.x; i < s.C; i += blockDim.x) {
    bs[i] = bias[i];
    sc[i] = fold[i];
    sh[i] = fold[s.C + i];
    mu[i] = fold[2 * s.C + i];
    iv[i] = fold[3 * s.C + i];
  }
  float a[CT], b[CT];
#pragma unroll
  for (int c = 0; c < CT; ++c) a[c] = b[c] = 0.f;
  const int HW = s.H * s.W, PW = s.W + 2;
  for (int n = blockIdx.x; n < s.B; n += gridDim.x) {
    __syncthreads();
    stage_image(X + (size_t)n * HW, xs, s.H, s.W);
    __syncthreads();
    const float* g = dF + (size_t)n * s.C * HW;
    for (int p = threadIdx.x; p < HW; p += blockDim.x) {
      float nb[9];
      load_patch(xs, p / s.W, p % s.W, PW, nb);
#pragma unroll
      for (int c = 0; c < CT; ++c) {
        if (c >= s.C) break;
        float z = conv_at(nb, ws + c * 9, bs[c]);
        float y = fmaf(z, sc[c], sh[c]);
        float dy = y > 0.f ? g[(size_t)c * HW + p] : 0.f;
        a[c] = fmaf(dy, (z - mu[c]) * iv[c], a[c]);
        b[c] += dy;
      }
    }
  }
  __syncthreads();
  reduce_to_global<CT>(a, b, s.C, bstats, bstats + s.C, red);
}

// dX, and dwb[0..9C) += d weights, dwb[9C..10C) += d bias.  With batch statistics
// dz = gamma/std * (dy - (d beta + zhat * d gamma) / count); with running statistics dz = gamma/std * dy.
template <int CT>
__global__ void __launch_bounds__(kThreads) conv_gate_bwd_apply(GateShape s, int training, double count,
                                                                const float* __restrict__ X,
                                                                const float* __restrict__ w,
                                                                const float* __restrict__ bias,
                                                                const float* __restrict__ fold,
                                                                const float* __restrict__ dF,
                                                                const double* __restrict__ bstats,
                                                                float* __restrict__ dX, double* __restrict__ dwb) {
  extern __shared__ float sm[];
  float* ws = sm;
  float* bs = ws + CT * 9;
  float* sc = bs + CT;
  float* sh = sc + CT;
  float* mu = sh + CT;
  float* iv = mu + CT;
  float* kg = iv + CT;    // d gamma / count
  float* kb = kg + CT;    // d beta / count
  float* red = kb + CT;
  float* xs = red + kThreads / 32;
  const int HW = s.H * s.W, PW = s.W + 2, plane = (s.H + 2) * PW;
  float* dzs = xs + plane;   // C bordered planes
  for (int i = threadIdx.x; i < s.C * 9; i += blockDim.x) ws[i] = w[i];
  for (int i = threadIdx.x; i < s.C; i += blockDim.x) {
    bs[i] = bias[i];
    sc[i] = fold[i];
    sh[i] = fold[s.C + i];
    mu[i] = fold[2 * s.C + i];
    iv[i] = fold[3 * s.C + i];
    kg[i] = training ? (float)(bstats[i] / count) : 0.f;
    kb[i] = training ? (float)(bstats[s.C + i] / count) : 0.f;
  }
  for (int i = threadIdx.x; i < s.C * plane; i += blockDim.x) dzs[i] = 0.f;   // the borders stay zero
  float aw[CT][9], ab[CT];
#pragma unroll
  for (int c = 0; c < CT; ++c) {
    ab[c] = 0.f;
#pragma unroll
    for (int t = 0; t < 9; ++t) aw[c][t] = 0.f;
  }
  for (int n = blockIdx.x; n < s.B; n += gridDim.x) {
    __syncthreads();
    stage_image(X + (size_t)n * HW, xs, s.H, s.W);
    __syncthreads();
    const float* g = dF + (size_t)n * s.C * HW;
    for (int p = threadIdx.x; p < HW; p += blockDim.x) {
      const int y = p / s.W, x = p % s.W;
      float nb[9];
      load_patch(xs, y, x, PW, nb);
#pragma unroll
      for (int c = 0; c < CT; ++c) {
        if (c >= s.C) break;
        float z = conv_at(nb, ws + c * 9, bs[c]);
        float zh = (z - mu[c]) * iv[c];
        float dy = fmaf(z, sc[c], sh[c]) > 0.f ? g[(size_t)c * HW + p] : 0.f;
        float dz = sc[c] * (dy - kb[c] - zh * kg[c]);
        dzs[c * plane + (y + 1) * PW + x + 1] = dz;
        ab[c] += dz;
#pragma unroll
        for (int t = 0; t < 9; ++t) aw[c][t] = fmaf(dz, nb[t], aw[c][t]);
      }
    }
    __syncthreads();
    for (int p = threadIdx.x; p < HW; p += blockDim.x) {
      const int y = p / s.W, x = p % s.W;
      float acc = 0.f;
      for (int c = 0; c < s.C; ++c) {
        const float* d = dzs + c * plane + (y + 2) * PW + x + 2;   // dz[y + 1 - i, x + 1 - j] in bordered coordinates
        const float* wc = ws + c * 9;
#pragma unroll
        for (int i = 0; i < 3; ++i)
#pragma unroll
          for (int j = 0; j < 3; ++j) acc = fmaf(wc[i * 3 + j], d[-i * PW - j], acc);
      }
      dX[(size_t)n * HW + p] = acc;
    }
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
  for (int c = 0; c < CT; ++c) {
    if (c >= s.C) break;
#pragma unroll
    for (int t = 0; t < 10; ++t) {
      float v = warp_sum(t < 9 ? aw[c][t < 9 ? t : 0] : ab[c]);
      if (lane == 0) red[warp] = v;
      __syncthreads();
      if (threadIdx.x == 0) {
        double tot = 0;
        for (int k = 0; k < nw; ++k) tot += red[k];
        atomicAdd(dwb + (t < 9 ? c * 9 + t : 9 * s.C + c), tot);
      }
      __syncthreads();
    }
  }
}

int grid_for(int B) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int g = sms * 4;
  return B < g ? B : g;
}

inline size_t plane_floats(int H, int W) { return (size_t)(H + 2) * (W + 2); }

template <int CT>
int forward_t(GateShape s, int training, const float* X, const float* w, const float* bias, const float* gamma,
              const float* beta, float* run_mean, float* run_var, float momentum, float eps, double* stats,
              float* fold, float* F, cudaStream_t st) {
  const int grid = grid_for(s.B);
  const double count = (double)s.B * s.H * s.W;
  if (training) {
    if (cudaMemsetAsync(stats, 0, 2 * s.C * sizeof(double), st) != cudaSuccess) return -4;
    size_t sm = (CT * 10 + 2 * (kThreads / 32) + plane_floats(s.H, s.W)) * sizeof(float);
    conv_gate_stats<CT><<<grid, kThreads, sm, st>>>(s, X, w, bias, stats);
  }
  conv_gate_finalize<<<1, 32, 0, st>>>(s.C, count, training, stats, gamma, beta, run_mean, run_var, momentum, eps, fold);
  size_t sm = (CT * 12 + plane_floats(s.H, s.W)) * sizeof(float);
  conv_gate_apply<CT><<<grid, kThreads, sm, st>>>(s, X, w, bias, fold, F);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

template <int CT>
int backward_t(GateShape s, int training, const float* X, const float* w, const float* bias, const float* fold,
               const float* dF, double* bstats, float* dX, double* dwb, cudaStream_t st) {
  const int grid = grid_for(s.B);
  const double count = (double)s.B * s.H * s.W;
  if (cudaMemsetAsync(bstats, 0, 2 * s.C * sizeof(double), st) != cudaSuccess) return -4;
  if (cudaMemsetAsync(dwb, 0, 10 * s.C * sizeof(double), st) != cudaSuccess) return -4;
  size_t sm1 = (CT * 14 + 2 * (kThreads / 32) + plane_floats(s.H, s.W)) * sizeof(float);
  conv_gate_bwd_stats<CT><<<grid, kThreads, sm1, st>>>(s, X, w, bias, fold, dF, bstats);
  size_t sm2 = (CT * 16 + kThreads / 32 + (size_t)(1 + s.C) * plane_floats(s.H, s.W)) * sizeof(float);
  conv_gate_bwd_apply<CT><<<grid, kThreads, sm2, st>>>(s, training, count, X, w, bias, fold, dF, bstats, dX, dwb);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

bool shape_ok(const GateShape& s) {
  if (s.B <= 0 || s.H <= 0 || s.W <= 0 || s.C <= 0 || s.C > 8) return false;
  return (16 * 8 + kThreads / 32 + (size_t)(1 + s.C) * plane_floats(s.H, s.W)) * sizeof(float) <= 48 * 1024;
}

}  // namespace

// 1 when the shape is covered (at most 8 channels, all bordered planes of one sample within 48 KB of shared memory).
extern "C" int dice_conv_gate_supported(int B, int H, int W, int C) { return shape_ok(GateShape{B, H, W, C}) ? 1 : 0; }

// X [B, H*W] fp32, w [C, 3, 3], bias [C], gamma / beta [C] (may be null), run_mean / run_var [C] (may be null when
// training), stats: 2C doubles of scratch, fold: 4C floats (kept for the backward pass), F [B, C*H*W].
extern "C" int dice_conv_gate_forward(int B, int H, int W, int C, int training, const float* X, const float* w,
                                      const float* bias, const float* gamma, const float* beta, float* run_mean,
                                      float* run_var, float momentum, float eps, double* stats, float* fold, float* F,
                                      void* stream) {
  GateShape s{B, H, W, C};
  if (!shape_ok(s)) return -1;
  if (!training && (run_mean == nullptr || run_var == nullptr)) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (C <= 2) return forward_t<2>(s, training, X, w, bias, gamma, beta, run_mean, run_var, momentum, eps, stats, fold, F, st);
  if (C <= 4) return forward_t<4>(s, training, X, w, bias, gamma, beta, run_mean, run_var, momentum, eps, stats, fold, F, st);
  return forward_t<8>(s, training, X, w, bias, gamma, beta, run_mean, run_var, momentum, eps, stats, fold, F, st);
}

// dF [B, C*H*W] -> dX [B, H*W]; bstats: 2C doubles (d gamma, d beta), dwb: 10C doubles (d weights, d bias).
extern "C" int dice_conv_gate_backward(int B, int H, int W, int C, int training, const float* X, const float* w,
                                       const float* bias, const float* fold, const float* dF, double* bstats,
                                       float* dX, double* dwb, void* stream) {
  GateShape s{B, H, W, C};
  if (!shape_ok(s)) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (C <= 2) return backward_t<2>(s, training, X, w, bias, fold, dF, bstats, dX, dwb, st);
  if (C <= 4) return backward_t<4>(s, training, X, w, bias, fold, dF, bstats, dX, dwb, st);
  return backward_t<8>(s, training, X, w, bias, fold, dF, bstats, dX, dwb, st);
}
