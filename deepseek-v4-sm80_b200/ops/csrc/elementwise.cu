// Bandwidth-bound row kernels: embedding gather, RMSNorm, FP8 activation quantisation, SwiGLU,
// RoPE, the fused q/kv norm+RoPE+QAT+cache-store, routed+shared add, argmax.
// All of them read each input once with 8/16-byte accesses and keep the row in registers.
#include "common.cuh"
#include "rope.cuh"

namespace {

__device__ __forceinline__ float block_sum(float v, float* sh) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float t = (l < nw) ? sh[l] : 0.f;
  t = warp_sum(t);
  return t;
}

// ------------------------------------------------------------------ embedding
// feedback != null: the token of row t is feedback[slots[t]] (the token sampled for that request by the previous
// step, which never left the device) and is also written to ids[t] for the kernels that need the id later.
__global__ void embed_kernel(int* __restrict__ ids, const int* __restrict__ feedback, const int* __restrict__ slots,
                             const uint4* __restrict__ w, uint4* __restrict__ out, int m, int h8) {
  pdl_entry();
  const int t = blockIdx.x;
  int id;
  if (feedback) {
    id = feedback[slots[t]];
    if (threadIdx.x == 0) ids[t] = id;
  } else {
    id = ids[t];
  }
  const uint4* src = w + (size_t)id * h8;
  for (int i = threadIdx.x; i < h8; i += blockDim.x) {
    const uint4 v = src[i];
    for (int s = 0; s < m; ++s) out[((size_t)t * m + s) * h8 + i] = v;
  }
}

// ------------------------------------------------------------------ RMSNorm (D <= 8192, D % 8 == 0)
__global__ void __launch_bounds__(256) rms_norm_kernel(const __nv_bfloat16* __restrict__ x, int ldx,
                                                       const __nv_bfloat16* __restrict__ w,
                                                       __nv_bfloat16* __restrict__ out, int ldo, int d, float eps,
                                                       uint8_t* __restrict__ q_out, float* __restrict__ s_out) {
  pdl_entry();
  __shared__ float sh[32];
  const int row = blockIdx.x;
  const __nv_bfloat16* xr = x + (size_t)row * ldx;
  float v[32];
  float ss = 0.f;
#pragma unroll
  for (int n = 0; n < 4; ++n) {
    const int i = (n * 256 + threadIdx.x) * 8;
    if (i < d) {
      const uint4 u = *reinterpret_cast<const uint4*>(xr + i);
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(p[k]);
        v[n * 8 + 2 * k] = f.x;
        v[n * 8 + 2 * k + 1] = f.y;
        ss += f.x * f.x + f.y * f.y;
      }
    }
  }
  ss = block_sum(ss, sh);
  const float r = rsqrtf(ss / d + eps);
#pragma unroll
  for (int n = 0; n < 4; ++n) {
    const int i = (n * 256 + threadIdx.x) * 8;
    if (i < d) {
      uint4 o;
      __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
      uint4 wu = make_uint4(0, 0, 0, 0);
      if (w) wu = *reinterpret_cast<const uint4*>(w + i);
      const __nv_bfloat162* pw = reinterpret_cast<const __nv_bfloat162*>(&wu);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float a = v[n * 8 + 2 * k] * r, b = v[n * 8 + 2 * k + 1] * r;
        if (w) {
          const float2 wf = __bfloat1622float2(pw[k]);
          a *= wf.x;
          b *= wf.y;
        }
        po[k] = __floats2bfloat162_rn(a, b);
      }
      *reinterpret_cast<uint4*>(out + (size_t)row * ldo + i) = o;
      if (q_out) {  // fused FP8 quantisation of the rounded result (needs d % 256 == 0: whole warps)
        float f[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 t = __bfloat1622float2(po[k]);
          f[2 * k] = t.x, f[2 * k + 1] = t.y;
        }
        quant8_store(f, q_out + (size_t)row * d, s_out + (size_t)row * (d / 128), i);
      }
    }
  }
}

// ------------------------------------------------------------------ FP8 activation quantisation
// scale = 2^ceil(log2(max(absmax, 1e-4) / 448)); q = e4m3_rn(clamp(x / scale)).  One warp per (row, block).
template <int BLOCK>
__global__ void fp8_quant_kernel(const __nv_bfloat16* __restrict__ x, int ldx, uint8_t* __restrict__ q,
                                 float* __restrict__ s, int rows, int k) {
  pdl_entry();
  constexpr int PER = BLOCK / 32;  // elements per lane: 4 (128) or 2 (64)
  const int nb = k / BLOCK;
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= rows * nb) return;
  const int row = gw / nb, b = gw % nb;
  const __nv_bfloat16* src = x + (size_t)row * ldx + b * BLOCK + lane * PER;
  float f[PER];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < PER; i += 2) {
    const float2 t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + i));
    f[i] = t.x;
    f[i + 1] = t.y;
    amax = fmaxf(amax, fmaxf(fabsf(t.x), fabsf(t.y)));
  }
  amax = warp_max(amax);
  const float sc = pow2_ceil_scale(amax);
  const float inv = 1.f / sc;  // exact: power of two
  uint8_t o[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const float c = fminf(fmaxf(f[i] * inv, -448.f), 448.f);
    o[i] = (uint8_t)__nv_cvt_float_to_fp8(c, __NV_SATFINITE, __NV_E4M3);
  }
  uint8_t* dst = q + (size_t)row * k + b * BLOCK + lane * PER;
  if (PER == 4)
    *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<uint32_t*>(o);
  else
    *reinterpret_cast<uint16_t*>(dst) = *reinterpret_cast<uint16_t*>(o);
  if (lane == 0) s[(size_t)row * nb + b] = sc;
}

// ------------------------------------------------------------------ SwiGLU with clamp: [T,2I] -> [T,I]
__global__ void silu_mul_clamp_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int rows,
                                      int inter, float limit) {
  pdl_entry();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t total = (size_t)rows * inter / 2;
  if (idx >= total) return;
  const int row = (int)(idx / (inter / 2)), c = (int)(idx % (inter / 2)) * 2;
  const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gu + (size_t)row * 2 * inter + c));
  const float2 u =
      __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gu + (size_t)row * 2 * inter + inter + c));
  float g0 = g.x, g1 = g.y, u0 = u.x, u1 = u.y;
  if (limit > 0.f) {
    g0 = fminf(g0, limit);
    g1 = fminf(g1, limit);
    u0 = fminf(fmaxf(u0, -limit), limit);
    u1 = fminf(fmaxf(u1, -limit), limit);
  }
  const float a0 = g0 / (1.f + expf(-g0)) * u0, a1 = g1 / (1.f + expf(-g1)) * u1;
  *reinterpret_cast<__nv_bfloat162*>(out + (size_t)row * inter + c) = __floats2bfloat162_rn(a0, a1);
}

// Same activation, 8 columns per thread, written only as e4m3 + block scales (the bf16 rounding of the activation
// is kept: the quantiser sees the rounded values).  inter % 128 == 0, so 16 consecutive threads share a block and
// every warp is whole.
__global__ void silu_mul_clamp_quant_kernel(const __nv_bfloat16* __restrict__ gu, uint8_t* __restrict__ q_out,
                                            float* __restrict__ s_out, int rows, int inter, float limit) {
  pdl_entry();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t total = (size_t)rows * inter / 8;
  if (idx >= total) return;  // total is a multiple of 16 per row and rows * inter / 8 of 32 when inter % 256 == 0
  const int row = (int)(idx / (inter / 8)), c = (int)(idx % (inter / 8)) * 8;
  const uint4 ug = *reinterpret_cast<const uint4*>(gu + (size_t)row * 2 * inter + c);
  const uint4 uu = *reinterpret_cast<const uint4*>(gu + (size_t)row * 2 * inter + inter + c);
  const __nv_bfloat162* pg = reinterpret_cast<const __nv_bfloat162*>(&ug);
  const __nv_bfloat162* pu = reinterpret_cast<const __nv_bfloat162*>(&uu);
  float f[8];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 g = __bfloat1622float2(pg[k]), u = __bfloat1622float2(pu[k]);
    float g0 = g.x, g1 = g.y, u0 = u.x, u1 = u.y;
    if (limit > 0.f) {
      g0 = fminf(g0, limit);
      g1 = fminf(g1, limit);
      u0 = fminf(fmaxf(u0, -limit), limit);
      u1 = fminf(fmaxf(u1, -limit), limit);
    }
    const float2 r = __bfloat1622float2(
        __floats2bfloat162_rn(g0 / (1.f + expf(-g0)) * u0, g1 / (1.f + expf(-g1)) * u1));
    f[2 * k] = r.x, f[2 * k + 1] = r.y;
  }
  quant8_store(f, q_out + (size_t)row * inter, s_out + (size_t)row * (inter / 128), c);
}

// ------------------------------------------------------------------ out = bf16(float(a) + float(b)); padded rows -> 0
__global__ void add_cast_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                __nv_bfloat16* __restrict__ out, int rows, int h, const int* __restrict__ num_valid) {
  pdl_entry();
  const size_t idx = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (idx >= (size_t)rows * h) return;
  const int row = (int)(idx / h);
  uint4 o = make_uint4(0, 0, 0, 0);
  if (!num_valid || row < *num_valid) {
    const uint4 ua = *reinterpret_cast<const uint4*>(a + idx), ub = *reinterpret_cast<const uint4*>(b + idx);
    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&ua);
    const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&ub);
    __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 fa = __bfloat1622float2(pa[k]), fb = __bfloat1622float2(pb[k]);
      po[k] = __floats2bfloat162_rn(fa.x + fb.x, fa.y + fb.y);
    }
  }
  *reinterpret_cast<uint4*>(out + idx) = o;
}

// ------------------------------------------------------------------ RoPE on the last R dims of [rows, D] (in place)
__global__ void rope_tail_kernel(__nv_bfloat16* __restrict__ x, const int* __restrict__ pos, int heads, int d,
                                 RopeParams rp, int inverse, int pos_offset) {
  pdl_entry();
  const int row = blockIdx.x;
  const int pair = threadIdx.x;
  if (pair >= rp.rotary_dim / 2) return;
  float c, s;
  rope_cos_sin(rp, (float)(pos[row / heads] + pos_offset), pair, inverse, c, s);
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(x + (size_t)row * d + (d - rp.rotary_dim)) + pair;
  const float2 v = __bfloat1622float2(*p);
  *p = __floats2bfloat162_rn(v.x * c - v.y * s, v.x * s + v.y * c);
}

// ------------------------------------------------------------------ q / kv norm + RoPE (+ QAT) + SWA store, D = 512
// blocks [0, T*H): one query head each (weightless RMSNorm + RoPE, in place);
// blocks [T*H, T*H+T): the token's kv row (RMSNorm*w + RoPE + block-64 e4m3 QAT on the 448 leading dims), written
// back in place and to the sliding-window cache row swa_map[loc / ps] * ps + loc % ps.
__global__ void __launch_bounds__(128) q_kv_norm_rope_store_kernel(
    __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ kv, int ldkv, const int* __restrict__ pos,
    const __nv_bfloat16* __restrict__ kvw, float eps, RopeParams rp, __nv_bfloat16* __restrict__ swa,
    const int* __restrict__ out_loc, const int* __restrict__ swa_map, int ps, int t_rows, int heads, int qat) {
  pdl_entry();
  constexpr int D = 512;
  __shared__ float sh[32];
  const int tid = threadIdx.x;
  const bool is_kv = blockIdx.x >= t_rows * heads;
  const int tok = is_kv ? blockIdx.x - t_rows * heads : blockIdx.x / heads;
  __nv_bfloat16* rowp = is_kv ? kv + (size_t)tok * ldkv : q + (size_t)blockIdx.x * D;
  float v[4];
  {
    const uint2 u = *reinterpret_cast<const uint2*>(rowp + tid * 4);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y;
  }
  float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
  ss = block_sum(ss, sh);
  const float r = rsqrtf(ss / D + eps);
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] *= r;
  if (is_kv) {
    const uint2 u = *reinterpret_cast<const uint2*>(kvw + tid * 4);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    v[0] *= a.x, v[1] *= a.y, v[2] *= b.x, v[3] *= b.y;
  }
  const int tail = D - rp.rotary_dim;
  if (tid * 4 >= tail) {
    const float p = (float)pos[tok];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float c, s;
      rope_cos_sin(rp, p, (tid * 4 - tail) / 2 + i, 0, c, s);
      const float a = v[2 * i], b = v[2 * i + 1];
      v[2 * i] = a * c - b * s;
      v[2 * i + 1] = a * s + b * c;
    }
  }
  __nv_bfloat162 o0 = __floats2bfloat162_rn(v[0], v[1]), o1 = __floats2bfloat162_rn(v[2], v[3]);
  if (is_kv && qat) {
    // 16 lanes cover one 64-wide group; the last 16 lanes (rope dims) keep their values
    const float2 f0 = __bfloat1622float2(o0), f1 = __bfloat1622float2(o1);
    float amax = fmaxf(fmaxf(fabsf(f0.x), fabsf(f0.y)), fmaxf(fabsf(f1.x), fabsf(f1.y)));
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (tid * 4 < tail) {
      const float sc = pow2_ceil_scale(amax), inv = 1.f / sc;
      float w[4] = {f0.x, f0.y, f1.x, f1.y};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float c = fminf(fmaxf(w[i] * inv, -448.f), 448.f);
        const __nv_fp8_storage_t e = __nv_cvt_float_to_fp8(c, __NV_SATFINITE, __NV_E4M3);
        w[i] = __half2float(__half(__nv_cvt_fp8_to_halfraw(e, __NV_E4M3))) * sc;
      }
      o0 = __floats2bfloat162_rn(w[0], w[1]);
      o1 = __floats2bfloat162_rn(w[2], w[3]);
    }
  }
  uint2 ou;
  ou.x = *reinterpret_cast<uint32_t*>(&o0);
  ou.y = *reinterpret_cast<uint32_t*>(&o1);
  *reinterpret_cast<uint2*>(rowp + tid * 4) = ou;
  if (is_kv) {
    const int loc = out_loc[tok];
    if (loc >= 0) {
      const int slot = swa_map[loc / ps];
      if (slot >= 0) *reinterpret_cast<uint2*>(swa + ((size_t)slot * ps + loc % ps) * D + tid * 4) = ou;
    }
  }
}

// ------------------------------------------------------------------ argmax over fp32 rows (lowest index wins ties)
__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ logits, long long* __restrict__ out,
                                                      int v) {
  pdl_entry();
  __shared__ float sv[32];
  __shared__ int si[32];
  const float* row = logits + (size_t)blockIdx.x * v;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < v; i += blockDim.x) {
    const float x = row[i];
    if (x > best || (x == best && i < bi)) best = x, bi = i;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ob > best || (ob == best && oi < bi)) best = ob, bi = oi;
  }
  if ((threadIdx.x & 31) == 0) sv[threadIdx.x >> 5] = best, si[threadIdx.x >> 5] = bi;
  __syncthreads();
  if (threadIdx.x < 32) {
    best = threadIdx.x < (blockDim.x >> 5) ? sv[threadIdx.x] : -INFINITY;
    bi = threadIdx.x < (blockDim.x >> 5) ? si[threadIdx.x] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) best = ob, bi = oi;
    }
    if (threadIdx.x == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
  }
}

// ------------------------------------------------------------------ index audit (checked runs)
// Every index the forward gathers with (token ids, cache locations, page-table entries, expert ids) can be audited
// before use: an entry outside [lo, hi) is recorded in the status word as DSV4_ERR_BAD_INDEX with the caller's tag and
// the entry's position, and nothing is dereferenced with it here.  The audited kernels themselves stay unchanged.
__global__ void index_check_kernel(const int* __restrict__ idx, long long n, int lo, int hi, int tag) {
  pdl_entry();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int v = idx[i];
    if (v < lo || v >= hi) dsv4_set_error(DSV4_ERR_BAD_INDEX, tag, (int)(i < 0x7fffffff ? i : 0x7fffffff));
  }
}

}  // namespace

DSV4_API int dsv4_embed(int* ids, const int* feedback, const int* slots, const void* w, void* out, int t, int m, int h,
                        cudaStream_t st) {
  if (t <= 0) return 0;
  if (h % 8 || (feedback && !slots)) return 120;
  dsv4_launch(embed_kernel, t, 256, 0, st, ids, feedback, slots, (const uint4*)w, (uint4*)out, m, h / 8);
  return (int)cudaGetLastError();
}
// q_out / s_out (may be null): additionally writes the e4m3 quantisation of the result, dense [rows, d] with one
// fp32 scale per 128 columns (needs d % 256 == 0).
DSV4_API int dsv4_rms_norm(const void* x, int ldx, const void* w, void* out, int ldo, int rows, int d, float eps,
                           void* q_out, float* s_out, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (d % 8 || d > 8192 || ldx % 8 || ldo % 8) return 121;
  if (q_out && (d % 256 || !s_out)) return 124;
  dsv4_launch(rms_norm_kernel, rows, 256, 0, st, (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w,
              (__nv_bfloat16*)out, ldo, d, eps, (uint8_t*)q_out, s_out);
  return (int)cudaGetLastError();
}
DSV4_API int dsv4_fp8_quant(const void* x, int ldx, void* q, float* s, int rows, int k, int block, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (k % block || (block != 128 && block != 64) || ldx % 4) return 122;
  const long long warps = (long long)rows * (k / block);
  const int blocks = (int)((warps * 32 + 255) / 256);
  if (block == 128)
    dsv4_launch(fp8_quant_kernel<128>, blocks, 256, 0, st, (const __nv_bfloat16*)x, ldx, (uint8_t*)q, s, rows, k);
  else
    dsv4_launch(fp8_quant_kernel<64>, blocks, 256, 0, st, (const __nv_bfloat16*)x, ldx, (uint8_t*)q, s, rows, k);
  return (int)cudaGetLastError();
}
// SwiGLU with clamp whose only output is the e4m3 quantisation (dense [rows, inter], one scale per 128 columns).
DSV4_API int dsv4_silu_mul_clamp_quant(const void* gu, void* q_out, float* s_out, int rows, int inter, float limit,
                                       cudaStream_t st) {
  if (rows <= 0) return 0;
  if (inter % 128) return 125;
  const size_t total = (size_t)rows * inter / 8;
  dsv4_launch(silu_mul_clamp_quant_kernel, (unsigned)((total + 255) / 256), 256, 0, st, (const __nv_bfloat16*)gu,
              (uint8_t*)q_out, s_out, rows, inter, limit);
  return (int)cudaGetLastError();
}
DSV4_API int dsv4_silu_mul_clamp(const void* gu, void* out, int rows, int inter, float limit, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (inter % 2) return 123;
  const size_t total = (size_t)rows * inter / 2;
  dsv4_launch(silu_mul_clamp_kernel, (unsigned)((total + 255) / 256), 256, 0, st, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out,
                                                                        rows, inter, limit);
  return (int)cudaGetLastError();
}
DSV4_API int dsv4_add_cast(const void* a, const void* b, void* out, int rows, int h, const int* num_valid,
                           cudaStream_t st) {
  if (rows <= 0) return 0;
  if (h % 8) return 124;
  const size_t total = (size_t)rows * h / 8;
  dsv4_launch(add_cast_kernel, (unsigned)((total + 255) / 256), 256, 0, st, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
                                                                  (__nv_bfloat16*)out, rows, h, num_valid);
  return (int)cudaGetLastError();
}
DSV4_API int dsv4_rope_tail(void* x, const int* pos, int rows, int heads, int d, RopeParams rp, int inverse,
                            int pos_offset, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (rp.rotary_dim > 128 || rp.rotary_dim % 2) return 125;
  dsv4_launch(rope_tail_kernel, rows, 64, 0, st, (__nv_bfloat16*)x, pos, heads, d, rp, inverse, pos_offset);
  return (int)cudaGetLastError();
}
DSV4_API int dsv4_q_kv_norm_rope_store(void* q, void* kv, int ldkv, const int* pos, const void* kvw, float eps,
                                       RopeParams rp, void* swa, const int* out_loc, const int* swa_map, int ps, int t,
                                       int heads, int d, int qat, cudaStream_t st) {
  if (t <= 0) return 0;
  if (d != 512 || rp.rotary_dim != 64 || ldkv % 4) return 126;
  dsv4_launch(q_kv_norm_rope_store_kernel, t * heads + t, 128, 0, st, (__nv_bfloat16*)q, (__nv_bfloat16*)kv, ldkv, pos,
                                                            (const __nv_bfloat16*)kvw, eps, rp, (__nv_bfloat16*)swa,
                                                            out_loc, swa_map, ps, t, heads, qat);
  return (int)cudaGetLastError();
}
DSV4_API int dsv4_argmax(const float* logits, long long* out, int rows, int v, cudaStream_t st) {
  if (rows <= 0) return 0;
  dsv4_launch(argmax_kernel, rows, 1024, 0, st, logits, out, v);
  return (int)cudaGetLastError();
}
// Audits n int32 indices against [lo, hi); see index_check_kernel.  tag identifies the audited tensor in the status word.
DSV4_API int dsv4_check_index(const int* idx, long long n, int lo, int hi, int tag, cudaStream_t st) {
  if (n <= 0) return 0;
  const long long blocks = (n + 255) / 256;
  dsv4_launch(index_check_kernel, (unsigned)(blocks < 1184 ? blocks : 1184), 256, 0, st, idx, n, lo, hi, tag);
  return (int)cudaGetLastError();
}
