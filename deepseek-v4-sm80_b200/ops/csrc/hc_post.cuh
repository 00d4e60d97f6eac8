// Hyper-connection "post" mix for 8 columns of one token, shared by hc.cu's consumers that fuse it behind a
// reduction (MoE combine, all-reduce):  xout[t, s, i..i+7] = post[s] * y + sum_j comb[j][s] * res[t, j, i..i+7],
// the arithmetic and fused-multiply-add order of hc_post_kernel (python/minisgl/kernel/triton/deepseek_v4.py:720 of
// the reference computes the same expression).
#pragma once
#include "common.cuh"

struct HcPostArgs {
  const __nv_bfloat16* res;  // [T, 4, h] residual streams (null: no post mix, plain output)
  const float* post;         // [T, 4]
  const float* comb;         // [T, 4, 4]
  __nv_bfloat16* xout;       // [T, 4, h]
};

__device__ __forceinline__ void hc_post_store8(const uint4& y8, const HcPostArgs& a, int t, int h, int i) {
  float yv[8], rv[4][8];
  const __nv_bfloat162* py = reinterpret_cast<const __nv_bfloat162*>(&y8);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 f = __bfloat1622float2(py[k]);
    yv[2 * k] = f.x, yv[2 * k + 1] = f.y;
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint4 u = *reinterpret_cast<const uint4*>(a.res + ((size_t)t * 4 + j) * h + i);
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(p[k]);
      rv[j][2 * k] = f.x, rv[j][2 * k + 1] = f.y;
    }
  }
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    const float ps = a.post[(size_t)t * 4 + s];
    uint4 o;
    __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float x0 = ps * yv[2 * k], x1 = ps * yv[2 * k + 1];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float c = a.comb[(size_t)t * 16 + j * 4 + s];
        x0 = fmaf(c, rv[j][2 * k], x0);
        x1 = fmaf(c, rv[j][2 * k + 1], x1);
      }
      po[k] = __floats2bfloat162_rn(x0, x1);
    }
    *reinterpret_cast<uint4*>(a.xout + ((size_t)t * 4 + s) * h + i) = o;
  }
}
