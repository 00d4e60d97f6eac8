// Rotary embedding parameters and the on-the-fly angle computation shared by every kernel that rotates.
// Interleaved pairs on the last `rotary_dim` dims, optional YaRN ramp, angle reduced to [-pi, pi) before
// cos/sin -- the arithmetic of the reference's kernels (python/minisgl/kernel/triton/deepseek_v4.py:97-141).
#pragma once
#include <cuda_runtime.h>

struct RopeParams {
  int rotary_dim;
  float log_base;
  int use_scaling;
  float factor;
  float low;
  float scale_denom;
};

__device__ __forceinline__ void rope_cos_sin(const RopeParams& rp, float pos, int pair, int inverse, float& c,
                                             float& s) {
  float inv = expf(-((2.0f * (float)pair) / (float)rp.rotary_dim) * rp.log_base);
  if (rp.use_scaling) {
    float ramp = ((float)pair - rp.low) / rp.scale_denom;
    ramp = fminf(fmaxf(ramp, 0.f), 1.f);
    const float smooth = 1.f - ramp;
    inv = inv / rp.factor * (1.f - smooth) + inv * smooth;
  }
  float theta = pos * inv;
  if (inverse) theta = -theta;
  theta = theta - floorf((theta + 3.141592653589793f) / 6.283185307179586f) * 6.283185307179586f;
  c = cosf(theta);
  s = sinf(theta);
}
