// KV compressors (ratio 4 with overlap, ratio 128 without) and the producers that publish their output:
//   compress_pool4 / compress_pool128 : softmax pooling at group boundaries from {rows of this call, the
//       per-request fp32 ring, the previous page's 4-row checkpoint}
//   compress_state4 / compress_state128 : carry this call's projected rows into ring / checkpoint
//   compress_store : pooled -> bf16 -> RMSNorm*w -> RoPE(pos+1-ratio) -> compressed cache row
//   indexer_kv_store : pooled -> norm -> RoPE -> Hadamard-128 -> power-of-two e4m3 row + scale
//   indexer_q_encode : indexer query RoPE + e4m3 with the scale folded into the per-head weight
// Semantics follow python/minisgl/kernel/triton/deepseek_v4.py:2419-2716 (C4), :2833-2975 (C128),
// :282-362 (store), :1095-1267 (indexer); the pooling is bit-stable across chunk boundaries because a group
// is always reduced in one pass at its boundary row, whatever mixture of sources supplies the rows.
#include "common.cuh"
#include "rope.cuh"

namespace {

__device__ __forceinline__ float pow2_ceil_scale_c(float amax) {
  const float v = __fdiv_rn(fmaxf(amax, 1e-4f), 448.f);
  const uint32_t b = __float_as_uint(v);
  const int e = (int)((b >> 23) & 0xff) - 127 + ((b & 0x7fffff) ? 1 : 0);
  return __uint_as_float((uint32_t)(e + 127) << 23);
}

// ------------------------------------------------------------------ C4 pooling
__global__ void compress_pool4_kernel(const float* __restrict__ proj, int ldp, const int* __restrict__ pos,
                                      const int* __restrict__ slots, const int* __restrict__ page_table, int ld_pt,
                                      const float* __restrict__ ring, const float* __restrict__ ckpt,
                                      const float* __restrict__ ape, float* __restrict__ out, int d, int ps) {
  pdl_entry();
  const int row = blockIdx.x;
  const int p = pos[row], s = slots[row];
  const int w4 = 4 * d;
  const bool boundary = ((p + 1) & 3) == 0;
  for (int f = threadIdx.x; f < d; f += blockDim.x) {
    if (!boundary) {
      out[(size_t)row * d + f] = 0.f;
      continue;
    }
    float kv[8], sc[8];
    float mx = -INFINITY;
#pragma unroll
    for (int src = 0; src < 8; ++src) {
      const int delta = 7 - src, lp = p - delta, cand = row - delta;
      const bool right = src >= 4;
      const int ko = right ? d : 0, so = right ? 3 * d : 2 * d;
      kv[src] = 0.f;
      sc[src] = -INFINITY;
      if (lp < 0) continue;
      const bool cur = cand >= 0 && slots[cand] == s && pos[cand] == lp;
      if (cur) {
        kv[src] = proj[(size_t)cand * ldp + ko + f];
        sc[src] = proj[(size_t)cand * ldp + so + f];
      } else if (!right && (lp / ps) != (p / ps)) {
        const int page = page_table[(size_t)s * ld_pt + lp] / ps;
        const float* c = ckpt + ((size_t)page * 4 + (lp & 3)) * 2 * d;
        kv[src] = c[f];
        sc[src] = c[d + f];
      } else {
        const float* r = ring + ((size_t)s * 8 + (lp & 7)) * w4;
        kv[src] = r[ko + f];
        sc[src] = r[so + f];
      }
      sc[src] += ape[(src & 3) * 2 * d + (right ? d : 0) + f];
      mx = fmaxf(mx, sc[src]);
    }
    float den = 0.f, acc = 0.f;
#pragma unroll
    for (int src = 0; src < 8; ++src) {
      const float w = expf(sc[src] - mx);
      den += w;
      acc += kv[src] * w;
    }
    out[(size_t)row * d + f] = acc / den;
  }
}

__global__ void compress_state4_kernel(const float* __restrict__ proj, int ldp, const int* __restrict__ pos,
                                       const int* __restrict__ slots, const int* __restrict__ page_table, int ld_pt,
                                       float* __restrict__ ring, float* __restrict__ ckpt, int d, int ps, int t_rows) {
  pdl_entry();
  const int row = blockIdx.x;
  const int p = pos[row], s = slots[row];
  const int w4 = 4 * d;
  const int later = row + 8;
  const bool overwritten = later < t_rows && slots[later] == s && pos[later] == p + 8;
  const float* src = proj + (size_t)row * ldp;
  if (!overwritten) {
    float* dst = ring + ((size_t)s * 8 + (p & 7)) * w4;
    for (int f = threadIdx.x; f < w4; f += blockDim.x) dst[f] = src[f];
  }
  if (p % ps >= ps - 4) {
    const int page = page_table[(size_t)s * ld_pt + p] / ps;
    float* c = ckpt + ((size_t)page * 4 + (p & 3)) * 2 * d;
    for (int f = threadIdx.x; f < d; f += blockDim.x) {
      c[f] = src[f];
      c[d + f] = src[2 * d + f];
    }
  }
}

// ------------------------------------------------------------------ C128 pooling (generic ratio without overlap)
__global__ void compress_pool128_kernel(const float* __restrict__ proj, int ldp, const int* __restrict__ pos,
                                        const int* __restrict__ slots, const float* __restrict__ ring,
                                        const float* __restrict__ ape, float* __restrict__ out, int d, int ratio) {
  pdl_entry();
  const int row = blockIdx.x;
  const int p = pos[row], s = slots[row];
  const int w2 = 2 * d;
  const bool boundary = ((p + 1) % ratio) == 0;
  extern __shared__ int cur_row[];  // [ratio]: row of this call supplying source i, or -1 (ring), or -2 (absent)
  for (int i = threadIdx.x; i < ratio; i += blockDim.x) {
    const int delta = ratio - 1 - i, lp = p - delta, cand = row - delta;
    int v = -1;
    if (lp < 0)
      v = -2;
    else if (cand >= 0 && slots[cand] == s && pos[cand] == lp)
      v = cand;
    cur_row[i] = v;
  }
  __syncthreads();
  for (int f = threadIdx.x; f < d; f += blockDim.x) {
    if (!boundary) {
      out[(size_t)row * d + f] = 0.f;
      continue;
    }
    // two passes (max, then weighted sum) keep the arithmetic identical to a plain softmax
    float mx = -INFINITY;
    for (int i = 0; i < ratio; ++i) {
      const int c = cur_row[i];
      if (c == -2) continue;
      const float scv = c >= 0 ? proj[(size_t)c * ldp + d + f] + ape[(size_t)i * d + f]
                               : ring[((size_t)s * ratio + i) * w2 + d + f];
      mx = fmaxf(mx, scv);
    }
    float den = 0.f, acc = 0.f;
    for (int i = 0; i < ratio; ++i) {
      const int c = cur_row[i];
      if (c == -2) continue;
      float kvv, scv;
      if (c >= 0) {
        kvv = proj[(size_t)c * ldp + f];
        scv = proj[(size_t)c * ldp + d + f] + ape[(size_t)i * d + f];
      } else {
        const float* r = ring + ((size_t)s * ratio + i) * w2;
        kvv = r[f];
        scv = r[d + f];
      }
      const float w = expf(scv - mx);
      den += w;
      acc += kvv * w;
    }
    out[(size_t)row * d + f] = acc / den;
  }
}

__global__ void compress_state128_kernel(const float* __restrict__ proj, int ldp, const int* __restrict__ pos,
                                         const int* __restrict__ slots, const float* __restrict__ ape,
                                         float* __restrict__ ring, int d, int ratio, int t_rows) {
  pdl_entry();
  const int row = blockIdx.x;
  const int p = pos[row], s = slots[row];
  const int later = row + ratio;
  if (later < t_rows && slots[later] == s && pos[later] == p + ratio) return;
  const int w2 = 2 * d, i = p % ratio;
  const float* src = proj + (size_t)row * ldp;
  float* dst = ring + ((size_t)s * ratio + i) * w2;
  for (int f = threadIdx.x; f < d; f += blockDim.x) {
    dst[f] = src[f];
    dst[d + f] = src[d + f] + ape[(size_t)i * d + f];
  }
}

// ------------------------------------------------------------------ pooled -> norm -> RoPE -> compressed cache (D = 512)
__global__ void __launch_bounds__(128) compress_store_kernel(const float* __restrict__ pooled,
                                                             const int* __restrict__ pos,
                                                             const int* __restrict__ out_loc,
                                                             const __nv_bfloat16* __restrict__ w, float eps,
                                                             RopeParams rp, __nv_bfloat16* __restrict__ cache, int ps,
                                                             int ratio) {
  pdl_entry();
  constexpr int D = 512;
  __shared__ float sh[4];
  const int row = blockIdx.x, tid = threadIdx.x;
  const int p = pos[row], loc = out_loc[row];
  if (((p + 1) % ratio) != 0 || loc < 0) return;
  float v[4];
  const float4 in = *reinterpret_cast<const float4*>(pooled + (size_t)row * D + tid * 4);
  v[0] = bf2f(f2bf(in.x)), v[1] = bf2f(f2bf(in.y)), v[2] = bf2f(f2bf(in.z)), v[3] = bf2f(f2bf(in.w));
  float ss = warp_sum(v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3]);
  if ((tid & 31) == 0) sh[tid >> 5] = ss;
  __syncthreads();
  const float r = rsqrtf((sh[0] + sh[1] + sh[2] + sh[3]) / D + eps);
  const uint2 wu = *reinterpret_cast<const uint2*>(w + tid * 4);
  const float2 w0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wu.x));
  const float2 w1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wu.y));
  v[0] *= r * w0.x, v[1] *= r * w0.y, v[2] *= r * w1.x, v[3] *= r * w1.y;
  const int tail = D - rp.rotary_dim;
  if (tid * 4 >= tail) {
    const float pp = (float)(p + 1 - ratio);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float c, s;
      rope_cos_sin(rp, pp, (tid * 4 - tail) / 2 + i, 0, c, s);
      const float a = v[2 * i], b = v[2 * i + 1];
      v[2 * i] = a * c - b * s;
      v[2 * i + 1] = a * s + b * c;
    }
  }
  const int rpp = ps / ratio > 0 ? ps / ratio : 1;
  const size_t crow = (size_t)(loc / ps) * rpp + (loc % ps) / ratio;
  __nv_bfloat162 o0 = __floats2bfloat162_rn(v[0], v[1]), o1 = __floats2bfloat162_rn(v[2], v[3]);
  uint2 ou;
  ou.x = *reinterpret_cast<uint32_t*>(&o0);
  ou.y = *reinterpret_cast<uint32_t*>(&o1);
  *reinterpret_cast<uint2*>(cache + crow * D + tid * 4) = ou;
}

// ------------------------------------------------------------------ indexer key row (D = 128), one warp per row
__global__ void indexer_kv_store_kernel(const float* __restrict__ pooled, const int* __restrict__ pos,
                                        const int* __restrict__ out_loc, const float* __restrict__ w, float eps,
                                        RopeParams rp, uint8_t* __restrict__ vals, float* __restrict__ scales, int ps,
                                        int t_rows) {
  pdl_entry();
  constexpr int D = 128;
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (row >= t_rows) return;
  const int p = pos[row], loc = out_loc[row];
  if (((p + 1) & 3) != 0 || loc < 0) return;
  float v[4];
  const float4 in = *reinterpret_cast<const float4*>(pooled + (size_t)row * D + lane * 4);
  v[0] = bf2f(f2bf(in.x)), v[1] = bf2f(f2bf(in.y)), v[2] = bf2f(f2bf(in.z)), v[3] = bf2f(f2bf(in.w));
  const float ss = warp_sum(v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3]);
  const float r = rsqrtf(ss / D + eps);
  const float4 wv = *reinterpret_cast<const float4*>(w + lane * 4);
  v[0] = bf2f(f2bf(v[0] * r * wv.x)), v[1] = bf2f(f2bf(v[1] * r * wv.y));
  v[2] = bf2f(f2bf(v[2] * r * wv.z)), v[3] = bf2f(f2bf(v[3] * r * wv.w));
  const int tail = D - rp.rotary_dim;
  if (lane * 4 >= tail) {
    const float pp = (float)(p - 3);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float c, s;
      rope_cos_sin(rp, pp, (lane * 4 - tail) / 2 + i, 0, c, s);
      const float a = v[2 * i], b = v[2 * i + 1];
      v[2 * i] = a * c - b * s;
      v[2 * i + 1] = a * s + b * c;
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = bf2f(f2bf(v[i]));
  // Walsh-Hadamard, element e = lane*4 + k: strides 1,2 in-thread, 4..64 across lanes
  {
    float a = v[0] + v[1], b = v[0] - v[1], c = v[2] + v[3], d2 = v[2] - v[3];
    v[0] = a + c, v[2] = a - c, v[1] = b + d2, v[3] = b - d2;
  }
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float o = __shfl_xor_sync(0xffffffffu, v[i], m);
      v[i] = (lane & m) ? (o - v[i]) : (v[i] + o);
    }
  }
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[i] = bf2f(f2bf(v[i] * 0.08838834764831845f));
    amax = fmaxf(amax, fabsf(v[i]));
  }
  amax = warp_max(amax);
  const float sc = pow2_ceil_scale_c(amax), inv = 1.f / sc;
  uint8_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    o[i] = (uint8_t)__nv_cvt_float_to_fp8(fminf(fmaxf(v[i] * inv, -448.f), 448.f), __NV_SATFINITE, __NV_E4M3);
  const size_t crow = (size_t)(loc / ps) * (ps / 4) + (loc % ps) / 4;
  *reinterpret_cast<uint32_t*>(vals + crow * D + lane * 4) = *reinterpret_cast<uint32_t*>(o);
  if (lane == 0) scales[crow] = sc;
}

// ------------------------------------------------------------------ indexer query (D = 128), one warp per (token, head)
__global__ void indexer_q_encode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ wts,
                                        const int* __restrict__ pos, RopeParams rp, float fold,
                                        uint8_t* __restrict__ codes, float* __restrict__ wout, int heads, int rows) {
  pdl_entry();
  constexpr int D = 128;
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int tok = row / heads;
  float v[4];
  {
    const uint2 u = *reinterpret_cast<const uint2*>(q + (size_t)row * D + lane * 4);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y;
  }
  const int tail = D - rp.rotary_dim;
  if (lane * 4 >= tail) {
    const float pp = (float)pos[tok];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float c, s;
      rope_cos_sin(rp, pp, (lane * 4 - tail) / 2 + i, 0, c, s);
      const float a = v[2 * i], b = v[2 * i + 1];
      v[2 * i] = a * c - b * s;
      v[2 * i + 1] = a * s + b * c;
    }
  }
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[i] = bf2f(f2bf(v[i]));
    amax = fmaxf(amax, fabsf(v[i]));
  }
  amax = warp_max(amax);
  const float sc = pow2_ceil_scale_c(amax), inv = 1.f / sc;
  uint8_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    o[i] = (uint8_t)__nv_cvt_float_to_fp8(fminf(fmaxf(v[i] * inv, -448.f), 448.f), __NV_SATFINITE, __NV_E4M3);
  *reinterpret_cast<uint32_t*>(codes + (size_t)row * D + lane * 4) = *reinterpret_cast<uint32_t*>(o);
  if (lane == 0) wout[row] = bf2f(wts[row]) * sc * fold;
}

}  // namespace

DSV4_API int dsv4_compress_pool(const float* proj, int ldp, const int* pos, const int* slots, const int* page_table, int ld_pt,
                                const float* ring, const float* ckpt, const float* ape, float* out, int t, int d,
                                int ratio, int ps, cudaStream_t st) {
  if (t <= 0) return 0;
  if (ratio == 4)
    dsv4_launch(compress_pool4_kernel, t, d < 256 ? d : 256, 0, st, proj, ldp, pos, slots, page_table, ld_pt, ring, ckpt, ape, out, d,
                                                          ps);
  else
    dsv4_launch(compress_pool128_kernel, t, d < 256 ? d : 256, ratio * sizeof(int), st, proj, ldp, pos, slots, ring, ape, out, d,
                                                                              ratio);
  return (int)cudaGetLastError();
}
DSV4_API int dsv4_compress_state(const float* proj, int ldp, const int* pos, const int* slots, const int* page_table, int ld_pt,
                                 float* ring, float* ckpt, const float* ape, int t, int d, int ratio, int ps,
                                 cudaStream_t st) {
  if (t <= 0) return 0;
  if (ratio == 4)
    dsv4_launch(compress_state4_kernel, t, 256, 0, st, proj, ldp, pos, slots, page_table, ld_pt, ring, ckpt, d, ps, t);
  else
    dsv4_launch(compress_state128_kernel, t, 256, 0, st, proj, ldp, pos, slots, ape, ring, d, ratio, t);
  return (int)cudaGetLastError();
}
DSV4_API int dsv4_compress_store(const float* pooled, const int* pos, const int* out_loc, const void* w, float eps,
                                 RopeParams rp, void* cache, int t, int d, int ps, int ratio, cudaStream_t st) {
  if (t <= 0) return 0;
  if (d != 512 || rp.rotary_dim != 64) return 140;
  dsv4_launch(compress_store_kernel, t, 128, 0, st, pooled, pos, out_loc, (const __nv_bfloat16*)w, eps, rp,
                                           (__nv_bfloat16*)cache, ps, ratio);
  return (int)cudaGetLastError();
}
DSV4_API int dsv4_indexer_kv_store(const float* pooled, const int* pos, const int* out_loc, const float* w, float eps,
                                   RopeParams rp, void* vals, float* scales, int t, int d, int ps, cudaStream_t st) {
  if (t <= 0) return 0;
  if (d != 128 || rp.rotary_dim != 64) return 141;
  dsv4_launch(indexer_kv_store_kernel, (t * 32 + 255) / 256, 256, 0, st, pooled, pos, out_loc, w, eps, rp, (uint8_t*)vals, scales,
                                                               ps, t);
  return (int)cudaGetLastError();
}
DSV4_API int dsv4_indexer_q_encode(const void* q, const void* wts, const int* pos, RopeParams rp, float fold,
                                   void* codes, float* wout, int t, int heads, int d, cudaStream_t st) {
  if (t <= 0) return 0;
  if (d != 128 || rp.rotary_dim != 64) return 142;
  const int rows = t * heads;
  dsv4_launch(indexer_q_encode_kernel, (rows * 32 + 255) / 256, 256, 0, st, (const __nv_bfloat16*)q, (const __nv_bfloat16*)wts,
                                                                  pos, rp, fold, (uint8_t*)codes, wout, heads, rows);
  return (int)cudaGetLastError();
}
