// Sparse-attention indexer: FP8 logits over a request's compressed (ratio 4) history and the deterministic top-k.
//
// logits[t, j] = k_scale[row_j] * sum_h relu(q[t,h,:] . k[row_j,:]) * w[t,h]   for j < (pos+1)/4, else -inf
// (python/minisgl/kernel/triton/deepseek_v4.py:1296-1384).  q and k are e4m3 codes; every product is exact in fp32.
// Each CTA owns one token and a 64-row slice of its history; a lane owns two heads, the key row is broadcast from
// shared memory, so there is one warp reduction per (token, row).
//
// top-k keeps the reference's contract (csrc/jit/dsv4_topk_v1.cu:275-479): rows shorter than k keep every entry,
// a non-finite score invalidates the row (len = -1), ties at the threshold are resolved towards the lower index.
// The selection is a 4-pass 8-bit radix select on order-preserving keys followed by an ordered compaction, so
// the result is deterministic and comes out sorted by index (attention does not depend on the order).
#include "common.cuh"

namespace {

constexpr int DI = 128;
constexpr int QLD = DI + 4;  // padded fp32 row stride: conflict-free 16-byte reads with lane = head

__device__ __forceinline__ float e4m3_to_float(uint8_t v) {
  return __half2float(__half(__nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)v, __NV_E4M3)));
}

__global__ void __launch_bounds__(256) indexer_logits_kernel(const uint8_t* __restrict__ qc, const float* __restrict__ wf,
                                                             const uint8_t* __restrict__ kvals,
                                                             const float* __restrict__ kscale,
                                                             const int* __restrict__ slots, const int* __restrict__ pos,
                                                             const int* __restrict__ page_table, int ld_pt, int ps,
                                                             float* __restrict__ logits, int width, int heads) {
  pdl_entry();
  extern __shared__ __align__(16) float ix_smem[];
  float* qs = ix_smem;                  // [heads][QLD]
  float* ks = qs + heads * QLD;         // [8 warps][DI]
  const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int j0 = blockIdx.y * 64;
  const int n = (pos[t] + 1) >> 2;
  if (j0 >= width) return;
  if (j0 >= n) {
    for (int j = j0 + tid; j < min(j0 + 64, width); j += 256) logits[(size_t)t * width + j] = -INFINITY;
    return;
  }
  for (int i = tid; i < heads * DI; i += 256) qs[(i / DI) * QLD + (i % DI)] = e4m3_to_float(qc[(size_t)t * heads * DI + i]);
  __syncthreads();
  const int* pt = page_table + (size_t)slots[t] * ld_pt;
  const int hpl = heads / 32;  // heads per lane (1 or 2)
  float w0 = wf[(size_t)t * heads + lane], w1 = hpl > 1 ? wf[(size_t)t * heads + lane + 32] : 0.f;
  float* kw = ks + warp * DI;
  for (int j = j0 + warp; j < min(j0 + 64, width); j += 8) {
    float out = -INFINITY;
    if (j < n) {
      const int loc = pt[4 * j + 3];
      const size_t row = (size_t)(loc / ps) * (ps / 4) + (loc % ps) / 4;
      const uint32_t kk = *reinterpret_cast<const uint32_t*>(kvals + row * DI + lane * 4);
      __syncwarp();
      kw[lane * 4 + 0] = e4m3_to_float(kk & 0xff);
      kw[lane * 4 + 1] = e4m3_to_float((kk >> 8) & 0xff);
      kw[lane * 4 + 2] = e4m3_to_float((kk >> 16) & 0xff);
      kw[lane * 4 + 3] = e4m3_to_float((kk >> 24) & 0xff);
      __syncwarp();
      float d0 = 0.f, d1 = 0.f;
      const float* q0 = qs + lane * QLD;
      const float* q1 = qs + (lane + 32) * QLD;
#pragma unroll 8
      for (int d = 0; d < DI; d += 4) {
        const float4 kv = *reinterpret_cast<const float4*>(kw + d);
        const float4 a = *reinterpret_cast<const float4*>(q0 + d);
        d0 = fmaf(a.x, kv.x, d0), d0 = fmaf(a.y, kv.y, d0), d0 = fmaf(a.z, kv.z, d0), d0 = fmaf(a.w, kv.w, d0);
        if (hpl > 1) {
          const float4 b = *reinterpret_cast<const float4*>(q1 + d);
          d1 = fmaf(b.x, kv.x, d1), d1 = fmaf(b.y, kv.y, d1), d1 = fmaf(b.z, kv.z, d1), d1 = fmaf(b.w, kv.w, d1);
        }
      }
      float s = fmaxf(d0, 0.f) * w0 + fmaxf(d1, 0.f) * w1;
      s = warp_sum(s);
      out = s * kscale[row];
    }
    if (lane == 0) logits[(size_t)t * width + j] = out;
  }
}

// ------------------------------------------------------------------ top-k
__device__ __forceinline__ uint32_t order_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ int block_excl_scan(int v, int* warp_tot, int& total) {
  // 1024 threads; returns exclusive prefix of v, total = block sum
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  int x = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  __syncthreads();
  if (lane == 31) warp_tot[w] = x;
  __syncthreads();
  if (w == 0) {
    int s = warp_tot[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, s, o);
      if (lane >= o) s += y;
    }
    warp_tot[lane] = s;
  }
  __syncthreads();
  total = warp_tot[31];
  return x - v + (w ? warp_tot[w - 1] : 0);
}

__global__ void __launch_bounds__(1024) topk_kernel(const float* __restrict__ logits, int width,
                                                    const int* __restrict__ pos, int* __restrict__ idx,
                                                    int* __restrict__ out_len, int k) {
  pdl_entry();
  __shared__ int hist[256];
  __shared__ int wt[32];
  __shared__ int sh_bad, sh_bin, sh_rem;
  const int t = blockIdx.x, tid = threadIdx.x;
  const int n = min((pos[t] + 1) >> 2, width);
  int* oi = idx + (size_t)t * k;
  if (n <= k) {
    for (int i = tid; i < k; i += 1024) oi[i] = i < n ? i : -1;
    if (tid == 0) out_len[t] = n;
    return;
  }
  const float* row = logits + (size_t)t * width;
  if (tid == 0) sh_bad = 0;
  __syncthreads();
  int bad = 0;
  for (int i = tid; i < n; i += 1024) bad |= !isfinite(row[i]);
  if (bad) sh_bad = 1;
  __syncthreads();
  if (sh_bad) {
    for (int i = tid; i < k; i += 1024) oi[i] = -1;
    if (tid == 0) out_len[t] = -1;
    return;
  }
  uint32_t prefix = 0, mask = 0;
  int rem = k;  // how many still to take among elements matching the prefix
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = tid; i < 256; i += 1024) hist[i] = 0;
    __syncthreads();
    for (int i = tid; i < n; i += 1024) {
      const uint32_t key = order_key(row[i]);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xff], 1);
    }
    __syncthreads();
    if (tid == 0) {
      int r = rem, b = 255;
      for (; b > 0; --b) {
        if (hist[b] >= r) break;
        r -= hist[b];
      }
      sh_bin = b;
      sh_rem = r;
    }
    __syncthreads();
    prefix |= (uint32_t)sh_bin << shift;
    mask |= 0xffu << shift;
    rem = sh_rem;
    __syncthreads();
  }
  // prefix = key of the k-th largest; take every key > prefix and the first `rem` (by index) equal to it
  int base = 0, eq_base = 0;
  for (int c = 0; c < n; c += 1024) {
    const int i = c + tid;
    uint32_t key = 0;
    if (i < n) key = order_key(row[i]);
    const int gt = i < n && key > prefix, eq = i < n && key == prefix;
    int eq_tot, sel_tot;
    const int eq_rank = eq_base + block_excl_scan(eq, wt, eq_tot);
    const int sel = gt || (eq && eq_rank < rem);
    const int p = base + block_excl_scan(sel, wt, sel_tot);
    if (sel && p < k) oi[p] = i;
    base += sel_tot;
    eq_base += eq_tot;
  }
  if (tid == 0) out_len[t] = k;
}

}  // namespace

DSV4_API int dsv4_indexer_logits(const void* qc, const float* wf, const void* kvals, const float* kscale,
                                 const int* slots, const int* pos, const int* page_table, int ld_pt, int ps,
                                 float* logits, int width, int t, int heads, int d, cudaStream_t st) {
  if (t <= 0 || width <= 0) return 0;
  if (d != DI || (heads != 32 && heads != 64)) return 400;
  const int smem = (heads * QLD + 8 * DI) * 4;
  dim3 grid(t, (width + 63) / 64);
  dsv4_launch(indexer_logits_kernel, grid, 256, smem, st, (const uint8_t*)qc, wf, (const uint8_t*)kvals, kscale, slots, pos,
                                                 page_table, ld_pt, ps, logits, width, heads);
  return (int)cudaGetLastError();
}

DSV4_API int dsv4_topk(const float* logits, int width, const int* pos, int* idx, int* out_len, int t, int k,
                       cudaStream_t st) {
  if (t <= 0) return 0;
  dsv4_launch(topk_kernel, t, 1024, 0, st, logits, width, pos, idx, out_len, k);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ allocation-free entry point (see noalloc.h)
#include "noalloc.h"

#include <stdio.h>

namespace {
// The logits workspace of the allocation-free entry point.  In host code this name is only a handle for the runtime
// (taking its address on the host does NOT give a device pointer); kernels get the address from cudaGetSymbolAddress.
static __device__ __align__(256) float g_noalloc_logits[DSV4_NOALLOC_MAX_ELEMS];
constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {};
thread_local char g_noalloc_err[256] = "";
}  // namespace

DSV4_API const char* dsv4_noalloc_last_error(void) { return g_noalloc_err; }

DSV4_API int dsv4_indexer_select_noalloc(const void* qc, const float* wf, const void* kvals, const float* kscale,
                                         const int* slots, const int* pos, const int* page_table, int ld_pt, int ps,
                                         int width, int t, int heads, int d, int* idx, int* out_len, int k,
                                         cudaStream_t stream) {
  g_noalloc_err[0] = 0;
  if (t <= 0) return 0;
  if (width <= 0 || (unsigned long long)t * (unsigned long long)width > DSV4_NOALLOC_MAX_ELEMS) {
    snprintf(g_noalloc_err, sizeof g_noalloc_err,
             "dsv4_indexer_select_noalloc: t * width = %d * %d exceeds the built-in workspace of %u floats; "
             "split the batch or use dsv4_indexer_logits + dsv4_topk with your own buffer",
             t, width, DSV4_NOALLOC_MAX_ELEMS);
    return 460;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    snprintf(g_noalloc_err, sizeof g_noalloc_err, "dsv4_indexer_select_noalloc: cannot identify the current device");
    return 461;
  }
  if (!g_noalloc_ptr[dev]) {  // once per device, with that device current
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_logits);
    if (e != cudaSuccess || !p) {
      snprintf(g_noalloc_err, sizeof g_noalloc_err, "dsv4_indexer_select_noalloc: cudaGetSymbolAddress failed: %s",
               cudaGetErrorString(e));
      return 461;
    }
    g_noalloc_ptr[dev] = p;
  }
  float* logits = g_noalloc_ptr[dev];
  int rc = dsv4_indexer_logits(qc, wf, kvals, kscale, slots, pos, page_table, ld_pt, ps, logits, width, t, heads, d,
                               stream);
  if (rc == 0) rc = dsv4_topk(logits, width, pos, idx, out_len, t, k, stream);
  if (rc != 0) snprintf(g_noalloc_err, sizeof g_noalloc_err, "dsv4_indexer_select_noalloc: launch failed with code %d", rc);
  return rc;
}
