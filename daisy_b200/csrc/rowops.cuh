// Per-row transforms on a 128-wide head vector held by a half-warp (16 lanes x 8 elements).
#pragma once
#include "common.cuh"

namespace daisy {

// Sum over the 16 lanes of a half-warp (lanes that differ in bits 0..3); all 16 get the result.
__device__ __forceinline__ float halfwarp_sum(float x) {
  x += __shfl_xor_sync(0xffffffffu, x, 8);
  x += __shfl_xor_sync(0xffffffffu, x, 4);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  return x;
}

// x[8] = elements 8*sub .. 8*sub+7 of one row (sub = lane & 15).  Applies the weightless RMS norm
// over the 128 elements and/or the half-rotation RoPE with the [64]-float table row cos_row/sin_row:
//   y[i]    =  x[i] cos[i] + x[i+64] sin[i]
//   y[i+64] = -x[i] sin[i] + x[i+64] cos[i]          (i < 64)
// All 32 lanes of the warp must call this together (shuffles).
__device__ __forceinline__ void norm_rope_row8(float* x, int sub, bool do_norm, bool do_rope, float eps,
                                               const float* __restrict__ cos_row, const float* __restrict__ sin_row) {
  if (do_norm) {
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += x[e] * x[e];
    ss = halfwarp_sum(ss);
    float r = rsqrtf(ss * (1.0f / DAISY_HEAD_DIM) + eps);
#pragma unroll
    for (int e = 0; e < 8; ++e) x[e] *= r;
  }
  if (do_rope) {
    const int f0 = 8 * (sub & 7);
    float4 c0 = *reinterpret_cast<const float4*>(cos_row + f0);
    float4 c1 = *reinterpret_cast<const float4*>(cos_row + f0 + 4);
    float4 s0 = *reinterpret_cast<const float4*>(sin_row + f0);
    float4 s1 = *reinterpret_cast<const float4*>(sin_row + f0 + 4);
    float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    const float sgn = (sub < 8) ? 1.f : -1.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float other = __shfl_xor_sync(0xffffffffu, x[e], 8);
      x[e] = x[e] * c[e] + sgn * other * s[e];
    }
  }
}

}  // namespace daisy
