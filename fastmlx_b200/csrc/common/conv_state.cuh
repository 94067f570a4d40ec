// What the mixers with a short causal convolution share: the kernel that moves a step's last inputs into a
// request's convolution state, and SiLU.
#pragma once
#include <math.h>
#include "common.cuh"

namespace {
constexpr int MAX_TAPS = 16;

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }

// One thread per (request, channel): the last taps-1 inputs of the request's portion (reaching back into the old
// state where the portion is shorter) become the new state.
template <typename T>
__global__ void conv_state_update_kernel(const T* proj, long long stride, const int* row_start, const int* row_slot,
                                         float* state, long long slot_stride, long long conv_off, int C, int taps,
                                         int max_slots) {
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int slot = row_slot[r];
  if (c >= C || slot < 0 || slot >= max_slots) return;
  const int first = row_start[r], n = row_start[r + 1] - first;
  float* cs = state + (long long)slot * slot_stride + conv_off;
  float keep[MAX_TAPS];
#pragma unroll
  for (int j = 0; j < MAX_TAPS; ++j) {
    if (j < taps - 1) {
      const int p = n - (taps - 1) + j;
      keep[j] = p >= 0 ? to_f(proj[(long long)(first + p) * stride + c]) : cs[(long long)(taps - 1 + p) * C + c];
    }
  }
#pragma unroll
  for (int j = 0; j < MAX_TAPS; ++j)
    if (j < taps - 1) cs[(long long)j * C + c] = keep[j];
}
}  // namespace
