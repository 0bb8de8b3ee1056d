// Multiplication tables of the bilinear score algebras (block layout: a row of width D is K blocks of width D / K)
// and the relation-normalisation modes, shared by the element-wise kernels.
#pragma once
#include <cuda_runtime.h>

namespace dice {

// ------------------------------------------------------------------------------------ algebra tables
// q_k = sum_a SGN[k][a] * h_a * r_{IDX[k][a]}   for K blocks of width D / K (block layout).
template <int K> struct Alg;
template <> struct Alg<1> {
  static __device__ __forceinline__ int idx(int k, int a) { return 0; }
  static __device__ __forceinline__ float sgn(int k, int a) { return 1.f; }
};
template <> struct Alg<2> {  // complex product
  static __device__ __forceinline__ int idx(int k, int a) { return k ^ a; }
  static __device__ __forceinline__ float sgn(int k, int a) { return (k == 0 && a == 1) ? -1.f : 1.f; }
};
template <> struct Alg<4> {  // Hamilton product
  static __device__ __forceinline__ int idx(int k, int a) { return k ^ a; }
  static __device__ __forceinline__ float sgn(int k, int a) {
    // rows k, columns a; entries are the sign of h_a * r_{k^a} in component k
    constexpr int S[4][4] = {{1, -1, -1, -1}, {1, 1, 1, -1}, {1, -1, 1, 1}, {1, 1, -1, 1}};
    return static_cast<float>(S[k][a]);
  }
};
template <> struct Alg<8> {  // octonion product
  static __device__ __forceinline__ int idx(int k, int a) { return k ^ a; }
  static __device__ __forceinline__ float sgn(int k, int a) {
    constexpr int S[8][8] = {{1, -1, -1, -1, -1, -1, -1, -1}, {1, 1, 1, -1, 1, -1, -1, 1},
                             {1, -1, 1, 1, 1, 1, -1, -1},     {1, 1, -1, 1, 1, -1, 1, -1},
                             {1, -1, -1, -1, 1, 1, 1, 1},     {1, 1, -1, 1, -1, 1, -1, 1},
                             {1, 1, 1, -1, -1, 1, 1, -1},     {1, -1, 1, 1, -1, -1, 1, 1}};
    return static_cast<float>(S[k][a]);
  }
};

enum NormMode : int { NORM_NONE = 0, NORM_ACROSS_BLOCKS = 1, NORM_CONSECUTIVE4 = 2 };

}  // namespace dice
