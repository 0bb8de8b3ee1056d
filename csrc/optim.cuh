// Element-wise update rules of the fused optimisers (Adam, AdamW, SGD, ADOPT), shared by the optimiser sweeps and by
// the scoring kernel, which applies them to an entity tile as soon as that tile's gradient is complete.
#pragma once
#include <cuda_runtime.h>

namespace dice {

// Step-dependent constants: bias corrections of Adam / AdamW, clip bound of ADOPT; t = number of this step (1-based).
struct OptStepConsts {
  float inv_bc1, inv_sqrt_bc2, clip;
  bool first_step;
};
__device__ __forceinline__ OptStepConsts opt_step_consts(int kind, long long t, float beta1, float beta2) {
  OptStepConsts c;
  c.inv_bc1 = 1.f;
  c.inv_sqrt_bc2 = 1.f;
  if (kind <= 1) {
    c.inv_bc1 = 1.f / (1.f - exp2f(static_cast<float>(t) * log2f(beta1)));
    c.inv_sqrt_bc2 = rsqrtf(1.f - exp2f(static_cast<float>(t) * log2f(beta2)));
  }
  c.clip = sqrtf(sqrtf(static_cast<float>(t - 1)));  // ADOPT: clip bound step^(1/4)
  c.first_step = (t == 1);
  return c;
}

// One parameter element: returns the updated weight; m / v are updated in place (registers).
__device__ __forceinline__ float opt_update(int kind, float w, float g, float& m, float& v, float lr, float beta1,
                                            float beta2, float eps, float wd, float inv_bc1, float inv_sqrt_bc2,
                                            float clip, bool first_step) {
  if (kind == 0) {
    g = fmaf(wd, w, g);
    m = fmaf(beta1, m, (1.f - beta1) * g);
    v = fmaf(beta2, v, (1.f - beta2) * g * g);
    return w - lr * inv_bc1 * m / (sqrtf(v) * inv_sqrt_bc2 + eps);
  } else if (kind == 1) {
    w *= 1.f - lr * wd;
    m = fmaf(beta1, m, (1.f - beta1) * g);
    v = fmaf(beta2, v, (1.f - beta2) * g * g);
    return w - lr * inv_bc1 * m / (sqrtf(v) * inv_sqrt_bc2 + eps);
  } else if (kind == 2) {
    g = fmaf(wd, w, g);
    return w - lr * g;
  }
  g = fmaf(wd, w, g);  // ADOPT
  if (first_step) {
    v = g * g;
    return w;
  }
  float ng = g / fmaxf(sqrtf(v), eps);
  ng = fminf(fmaxf(ng, -clip), clip);
  m = m + (1.f - beta1) * (ng - m);
  v = fmaf(beta2, v, (1.f - beta2) * g * g);
  return w - lr * m;
}

}  // namespace dice
