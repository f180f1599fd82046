// Register-resident top-k list shared by the router kernels.
#pragma once
#include <cuda_runtime.h>
#include <math_constants.h>

namespace b200 {

constexpr int ROUTER_MAX_K = 8;

// Keeps the largest (value, index) pairs seen so far in descending order.
struct TopK {
  float v[ROUTER_MAX_K];
  int i[ROUTER_MAX_K];
  __device__ __forceinline__ void init() {
#pragma unroll
    for (int j = 0; j < ROUTER_MAX_K; ++j) { v[j] = -CUDART_INF_F; i[j] = -1; }
  }
  // Candidates must arrive in increasing index order: a strict comparison then
  // keeps the lower index ahead on ties.
  __device__ __forceinline__ void push(float x, int idx) {
    float cv = x;
    int ci = idx;
#pragma unroll
    for (int j = 0; j < ROUTER_MAX_K; ++j) {
      if (cv > v[j]) {
        const float tv = v[j]; const int ti = i[j];
        v[j] = cv; i[j] = ci;
        cv = tv; ci = ti;
      }
    }
  }
};

}  // namespace b200
