// Small single-CTA reductions shared by the loss operators (fixed summation order).
#pragma once
#include "common.cuh"

namespace hilda {

// *out = number of targets != ignore_index
static __global__ void __launch_bounds__(1024)
count_valid_kernel(const int64_t* __restrict__ targets, int64_t n, int64_t ignore_index, int* __restrict__ out) {
  __shared__ int red[32];
  int c = 0;
  for (int64_t i = threadIdx.x; i < n; i += 1024) c += (targets[i] != ignore_index) ? 1 : 0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x < 32) {
    c = red[threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
    if (threadIdx.x == 0) *out = c;
  }
}

// *out = sum(rows) / (divide ? max(*n_valid, 1) : 1)
static __global__ void __launch_bounds__(1024)
sum_rows_kernel(const float* __restrict__ rows, int64_t n, const int* __restrict__ n_valid, int divide,
                float* __restrict__ out) {
  __shared__ float red[33];
  float acc = 0.f;
  for (int64_t i = threadIdx.x; i < n; i += 1024) acc += rows[i];
  acc = block_sum<1024>(acc, red);
  if (threadIdx.x == 0) {
    if (divide) acc /= fmaxf((float)(*n_valid), 1.0f);
    *out = acc;
  }
}

}  // namespace hilda
