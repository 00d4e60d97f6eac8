// Hyper-connection mixing (4 residual streams).
//
// hc_pre:  one CTA per token fuses what the reference runs as a cuBLAS GEMM plus two Triton kernels plus the
//          following RMSNorm (python/minisgl/kernel/triton/deepseek_v4.py:773-923, host :3765):
//          mixes = flatten(x) . fn^T (bf16 products, fp32 accumulate), r = rsqrt(mean(x^2)+eps),
//          pre = sigmoid(.)+eps, post = 2 sigmoid(.), comb = sinkhorn(softmax(.)+eps), y = sum_i pre_i x_i,
//          then optionally RMSNorm(y) * w.  The token's 4 x H row is staged once in shared memory.
// hc_head: same with 4 mix rows and only the `pre` branch (final stream collapse).
// hc_post: out_i = post_i * y + sum_j comb[j][i] * residual_j.
#include "common.cuh"

namespace {

constexpr int kM = 4;  // streams

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }

template <int MIX>  // 24 = layer (pre, post, comb), 4 = head (pre only)
__global__ void __launch_bounds__(256) hc_pre_kernel(const __nv_bfloat16* __restrict__ x,
                                                     const __nv_bfloat16* __restrict__ fn,
                                                     const float* __restrict__ mixes_in, int ld_mix, int n_part,
                                                     long long part_stride,
                                                     const float* __restrict__ scale, const float* __restrict__ base,
                                                     const __nv_bfloat16* __restrict__ norm_w,
                                                     __nv_bfloat16* __restrict__ y, float* __restrict__ post,
                                                     float* __restrict__ comb, int h, int iters, float eps,
                                                     float norm_eps, float rms_eps, uint8_t* __restrict__ q_out,
                                                     float* __restrict__ s_out) {
  pdl_entry();
  extern __shared__ __align__(16) uint8_t hc_smem[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(hc_smem);  // [4*h]
  __shared__ float red[32];
  __shared__ float mixes[MIX];
  __shared__ float pre_s[kM];
  const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int total = kM * h;
  const __nv_bfloat16* xr = x + (size_t)t * total;
  float ss = 0.f;
  for (int i = tid * 8; i < total; i += 256 * 8) {
    const uint4 u = *reinterpret_cast<const uint4*>(xr + i);
    *reinterpret_cast<uint4*>(xs + i) = u;
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(p[k]);
      ss += f.x * f.x + f.y * f.y;
    }
  }
  ss = warp_sum(ss);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  // mix rows: taken from a tensor-core GEMM over all tokens when the caller ran one (every CTA re-reading the
  // [MIX, 4h] matrix costs more than the rest of the kernel), else warp w computes rows w, w+8, ...
  if (mixes_in) {
    // split-K partial products: warp w adds splits w, w + 8, ..., then the eight sums are added in warp order
    // (a fixed tree, so the result does not depend on timing)
    __shared__ float part_s[8][32];
    float a = 0.f;
    for (int p0 = warp; p0 < n_part; p0 += 64) {  // eight loads in flight per thread
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int p = p0 + 8 * u;
        v[u] = (lane < MIX && p < n_part) ? __ldg(mixes_in + (size_t)p * part_stride + (size_t)t * ld_mix + lane) : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) a += v[u];
    }
    part_s[warp][lane] = a;
    __syncthreads();
    if (tid < MIX) {
      float m = 0.f;
#pragma unroll
      for (int w8 = 0; w8 < 8; ++w8) m += part_s[w8][tid];
      mixes[tid] = m;
    }
  } else
  for (int r = warp; r < MIX; r += 8) {
    const __nv_bfloat16* fr = fn + (size_t)r * total;
    float acc = 0.f;
    for (int i = lane * 8; i < total; i += 32 * 8) {
      const uint4 uf = *reinterpret_cast<const uint4*>(fr + i);
      const uint4 ux = *reinterpret_cast<const uint4*>(xs + i);
      const __nv_bfloat162* pf = reinterpret_cast<const __nv_bfloat162*>(&uf);
      const __nv_bfloat162* px = reinterpret_cast<const __nv_bfloat162*>(&ux);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 a = __bfloat1622float2(pf[k]), b = __bfloat1622float2(px[k]);
        acc = fmaf(a.x, b.x, acc);
        acc = fmaf(a.y, b.y, acc);
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) mixes[r] = acc;
  }
  __syncthreads();
  if (warp == 0) {
    float tot = (lane < 8) ? red[lane] : 0.f;
    tot = warp_sum(tot);
    const float r = rsqrtf(tot / (float)total + norm_eps);
    if (lane < kM) {
      const float pre = sigmoidf_(mixes[lane] * r * scale[0] + base[lane]) + eps;
      pre_s[lane] = pre;
      if (MIX == 24) post[(size_t)t * kM + lane] = 2.f * sigmoidf_(mixes[kM + lane] * r * scale[1] + base[kM + lane]);
    }
    if (MIX == 24) {
      // lanes 0..15 hold comb[j][i] with j = lane / 4 (row), i = lane % 4 (column)
      const int l16 = lane & 15;
      float v = mixes[2 * kM + l16] * r * scale[2] + base[2 * kM + l16];
      float mx = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      float e = expf(v - mx);
      float rs = e + __shfl_xor_sync(0xffffffffu, e, 1);
      rs += __shfl_xor_sync(0xffffffffu, rs, 2);
      float c = e / fmaxf(rs, eps) + eps;
      float cs = c + __shfl_xor_sync(0xffffffffu, c, 4);
      cs += __shfl_xor_sync(0xffffffffu, cs, 8);
      c = c / (cs + eps);
      for (int it = 0; it < iters - 1; ++it) {
        rs = c + __shfl_xor_sync(0xffffffffu, c, 1);
        rs += __shfl_xor_sync(0xffffffffu, rs, 2);
        c = c / (rs + eps);
        cs = c + __shfl_xor_sync(0xffffffffu, c, 4);
        cs += __shfl_xor_sync(0xffffffffu, cs, 8);
        c = c / (cs + eps);
      }
      if (lane < 16) comb[(size_t)t * 16 + lane] = c;
    }
  }
  __syncthreads();
  const float p0 = pre_s[0], p1 = pre_s[1], p2 = pre_s[2], p3 = pre_s[3];
  // y = sum_i pre_i x_i, rounded to bf16; then optional RMSNorm on the rounded values
  float yv[16];
  float ys = 0.f;
#pragma unroll
  for (int n = 0; n < 2; ++n) {
    const int i = (n * 256 + tid) * 8;
    if (i < h) {
      const uint4 u0 = *reinterpret_cast<const uint4*>(xs + i), u1 = *reinterpret_cast<const uint4*>(xs + h + i);
      const uint4 u2 = *reinterpret_cast<const uint4*>(xs + 2 * h + i),
                  u3 = *reinterpret_cast<const uint4*>(xs + 3 * h + i);
      const __nv_bfloat162* a0 = reinterpret_cast<const __nv_bfloat162*>(&u0);
      const __nv_bfloat162* a1 = reinterpret_cast<const __nv_bfloat162*>(&u1);
      const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&u2);
      const __nv_bfloat162* a3 = reinterpret_cast<const __nv_bfloat162*>(&u3);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f0 = __bfloat1622float2(a0[k]), f1 = __bfloat1622float2(a1[k]);
        const float2 f2 = __bfloat1622float2(a2[k]), f3 = __bfloat1622float2(a3[k]);
        const float s0 = p0 * f0.x + p1 * f1.x + p2 * f2.x + p3 * f3.x;
        const float s1 = p0 * f0.y + p1 * f1.y + p2 * f2.y + p3 * f3.y;
        const float2 rr = __bfloat1622float2(__floats2bfloat162_rn(s0, s1));
        yv[n * 8 + 2 * k] = rr.x;
        yv[n * 8 + 2 * k + 1] = rr.y;
        ys += rr.x * rr.x + rr.y * rr.y;
      }
    }
  }
  float rn = 1.f;
  if (norm_w) {
    ys = warp_sum(ys);
    __syncthreads();
    if (lane == 0) red[warp] = ys;
    __syncthreads();
    float tot = (lane < 8) ? red[lane] : 0.f;
    tot = warp_sum(tot);
    rn = rsqrtf(tot / (float)h + rms_eps);
  }
#pragma unroll
  for (int n = 0; n < 2; ++n) {
    const int i = (n * 256 + tid) * 8;
    if (i < h) {
      uint4 o;
      __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
      uint4 wu = make_uint4(0, 0, 0, 0);
      if (norm_w) wu = *reinterpret_cast<const uint4*>(norm_w + i);
      const __nv_bfloat162* pw = reinterpret_cast<const __nv_bfloat162*>(&wu);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float a = yv[n * 8 + 2 * k], b = yv[n * 8 + 2 * k + 1];
        if (norm_w) {
          const float2 wf = __bfloat1622float2(pw[k]);
          a = a * rn * wf.x;
          b = b * rn * wf.y;
        }
        po[k] = __floats2bfloat162_rn(a, b);
      }
      *reinterpret_cast<uint4*>(y + (size_t)t * h + i) = o;
      if (q_out) {  // fused FP8 quantisation of the rounded result (h % 256 == 0: whole warps)
        float f[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 tt = __bfloat1622float2(po[k]);
          f[2 * k] = tt.x, f[2 * k + 1] = tt.y;
        }
        quant8_store(f, q_out + (size_t)t * h, s_out + (size_t)t * (h / 128), i);
      }
    }
  }
}

__global__ void __launch_bounds__(256) hc_post_kernel(const __nv_bfloat16* __restrict__ y,
                                                      const __nv_bfloat16* __restrict__ res,
                                                      const float* __restrict__ post, const float* __restrict__ comb,
                                                      __nv_bfloat16* __restrict__ out, int h) {
  pdl_entry();
  const int t = blockIdx.x;
  const int i = (blockIdx.y * 256 + threadIdx.x) * 8;
  __shared__ float ps[kM], cs[16];
  if (threadIdx.x < kM) ps[threadIdx.x] = post[(size_t)t * kM + threadIdx.x];
  if (threadIdx.x < 16) cs[threadIdx.x] = comb[(size_t)t * 16 + threadIdx.x];
  __syncthreads();
  if (i >= h) return;
  float yv[8], rv[kM][8];
  {
    const uint4 u = *reinterpret_cast<const uint4*>(y + (size_t)t * h + i);
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(p[k]);
      yv[2 * k] = f.x, yv[2 * k + 1] = f.y;
    }
  }
#pragma unroll
  for (int j = 0; j < kM; ++j) {
    const uint4 u = *reinterpret_cast<const uint4*>(res + ((size_t)t * kM + j) * h + i);
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(p[k]);
      rv[j][2 * k] = f.x, rv[j][2 * k + 1] = f.y;
    }
  }
#pragma unroll
  for (int s = 0; s < kM; ++s) {
    uint4 o;
    __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float a = ps[s] * yv[2 * k], b = ps[s] * yv[2 * k + 1];
#pragma unroll
      for (int j = 0; j < kM; ++j) {
        a = fmaf(cs[j * kM + s], rv[j][2 * k], a);
        b = fmaf(cs[j * kM + s], rv[j][2 * k + 1], b);
      }
      po[k] = __floats2bfloat162_rn(a, b);
    }
    *reinterpret_cast<uint4*>(out + ((size_t)t * kM + s) * h + i) = o;
  }
}

}  // namespace

// mix_rows = 24: writes y, post, comb.  mix_rows = 4: head collapse (post/comb unused).  norm_w may be null.
// mixes (may be null): n_part split-K partial products of x_flat . fn^T from a GEMM over all tokens, fp32
// [n_part][t, ld_mix] spaced part_stride floats apart; the kernel adds them in order.  When null it computes the
// products itself.
DSV4_API int dsv4_hc_pre(const void* x, const void* fn, const float* mixes, int ld_mix, int n_part,
                         long long part_stride, const float* scale,
                         const float* base, const void* norm_w,
                         void* y, float* post, float* comb, int t, int h, int mix_rows, int iters, float eps,
                         float norm_eps, float rms_eps, void* q_out, float* s_out, cudaStream_t st) {
  if (t <= 0) return 0;
  if (h % 8 || h > 4096) return 130;
  if (q_out && (h % 256 || !s_out)) return 133;
  const int smem = kM * h * 2;
  if (mix_rows == 24) {
    static bool set = false;
    if (!set) {
      cudaFuncSetAttribute(hc_pre_kernel<24>, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * 4096 * 2);
      set = true;
    }
    dsv4_launch(hc_pre_kernel<24>, t, 256, smem, st, (const __nv_bfloat16*)x, (const __nv_bfloat16*)fn, mixes, ld_mix, n_part, part_stride, scale, base,
                                           (const __nv_bfloat16*)norm_w, (__nv_bfloat16*)y, post, comb, h, iters, eps,
                                           norm_eps, rms_eps, (uint8_t*)q_out, s_out);
  } else if (mix_rows == 4) {
    static bool set4 = false;
    if (!set4) {
      cudaFuncSetAttribute(hc_pre_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * 4096 * 2);
      set4 = true;
    }
    dsv4_launch(hc_pre_kernel<4>, t, 256, smem, st, (const __nv_bfloat16*)x, (const __nv_bfloat16*)fn, mixes, ld_mix, n_part, part_stride, scale, base,
                                          (const __nv_bfloat16*)norm_w, (__nv_bfloat16*)y, post, comb, h, iters, eps,
                                          norm_eps, rms_eps, (uint8_t*)q_out, s_out);
  } else {
    return 131;
  }
  return (int)cudaGetLastError();
}

DSV4_API int dsv4_hc_post(const void* y, const void* res, const float* post, const float* comb, void* out, int t, int h,
                          cudaStream_t st) {
  if (t <= 0) return 0;
  if (h % 8) return 132;
  dim3 grid(t, (h / 8 + 255) / 256);
  dsv4_launch(hc_post_kernel, grid, 256, 0, st, (const __nv_bfloat16*)y, (const __nv_bfloat16*)res, post, comb,
                                       (__nv_bfloat16*)out, h);
  return (int)cudaGetLastError();
}
