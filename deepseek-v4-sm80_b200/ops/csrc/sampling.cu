// Temperature / top-k / top-p sampling, one CTA per request row, replacing the reference's flashinfer calls
// (python/minisgl/engine/sample.py:69-90).
//
// Definition (the PyTorch oracle implements the same one): p = softmax(logits / T).  Order the vocabulary by
// (p descending, id ascending); entry of rank r is kept iff (top_k <= 0 or r < top_k) and the probability mass
// before it is < top_p.  The sample is the first kept id, in id order, whose running kept mass reaches
// u * kept_mass.  Rows with T <= 0 or top_k == 1 are greedy (lowest id among the maxima).
// Masses are accumulated as 2^-40 fixed point so that every reduction is order independent: the same logits
// and u always give the same token.  An optional mask adds -inf to given ids first (reasoning sampler).
#include "common.cuh"

namespace {

__device__ __forceinline__ uint32_t okey(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ unsigned long long fx(float p) { return (unsigned long long)((double)p * 1099511627776.0); }

__device__ __forceinline__ unsigned long long block_scan_u64(unsigned long long v, unsigned long long* wt,
                                                             unsigned long long& total) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  unsigned long long x = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  __syncthreads();
  if (lane == 31) wt[w] = x;
  __syncthreads();
  if (w == 0) {
    unsigned long long s = wt[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long y = __shfl_up_sync(0xffffffffu, s, o);
      if (lane >= o) s += y;
    }
    wt[lane] = s;
  }
  __syncthreads();
  total = wt[31];
  return x - v + (w ? wt[w - 1] : 0ull);
}

__global__ void __launch_bounds__(1024) sample_kernel(const float* __restrict__ logits, int v,
                                                      const float* __restrict__ temperature,
                                                      const int* __restrict__ top_k, const float* __restrict__ top_p,
                                                      const float* __restrict__ uniform,
                                                      const int* __restrict__ mask_ids, int n_mask,
                                                      long long* __restrict__ out) {
  pdl_entry();
  __shared__ float sf[32];
  __shared__ int si[32];
  __shared__ unsigned long long wt[32];
  __shared__ unsigned long long hmass[256];
  __shared__ int hcnt[256];
  __shared__ int sh_bin, sh_cnt_above;
  __shared__ unsigned long long sh_mass_above;
  const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const float* row = logits + (size_t)b * v;
  const int* mrow = mask_ids ? mask_ids + (size_t)b * n_mask : nullptr;
  auto val = [&](int i) -> float {
    float x = row[i];
    for (int m = 0; m < n_mask; ++m)
      if (mrow[m] == i) x = -INFINITY;
    return x;
  };
  // argmax (lowest id wins ties) -- also the softmax max
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = tid; i < v; i += 1024) {
    const float x = val(i);
    if (x > best || (x == best && i < bi)) best = x, bi = i;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ob > best || (ob == best && oi < bi)) best = ob, bi = oi;
  }
  if (lane == 0) sf[w] = best, si[w] = bi;
  __syncthreads();
  if (w == 0) {
    best = sf[lane], bi = si[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) best = ob, bi = oi;
    }
    if (lane == 0) sf[0] = best, si[0] = bi;
  }
  __syncthreads();
  const float mx = sf[0];
  const int amax = si[0];
  const float temp = temperature ? temperature[b] : 0.f;
  const int tk = top_k ? top_k[b] : -1;
  const float tp = top_p ? top_p[b] : 1.f;
  if (temp <= 0.f || tk == 1) {
    if (tid == 0) out[b] = amax;
    return;
  }
  const float inv_t = 1.f / temp;
  // Z in fixed point of exp((x - mx)/T)  (each term <= 1)
  unsigned long long zl = 0;
  for (int i = tid; i < v; i += 1024) zl += fx(expf((val(i) - mx) * inv_t));
  unsigned long long ztot;
  block_scan_u64(zl, wt, ztot);
  const unsigned long long p_limit = tp >= 1.f ? ~0ull : (unsigned long long)((double)ztot * (double)tp);
  const int k_limit = tk > 0 ? tk : 0x7fffffff;
  // radix descent: find the key of the last kept rank
  uint32_t prefix = 0, mask = 0;
  int cnt_above = 0;
  unsigned long long mass_above = 0;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = tid; i < 256; i += 1024) hcnt[i] = 0, hmass[i] = 0ull;
    __syncthreads();
    for (int i = tid; i < v; i += 1024) {
      const float x = val(i);
      const uint32_t key = okey(x);
      if ((key & mask) == prefix) {
        atomicAdd(&hcnt[(key >> shift) & 0xff], 1);
        atomicAdd(&hmass[(key >> shift) & 0xff], fx(expf((x - mx) * inv_t)));
      }
    }
    __syncthreads();
    if (tid == 0) {
      int c = cnt_above, bsel = 0;
      unsigned long long m = mass_above;
      for (int bb = 255; bb >= 0; --bb) {
        // does the kept set end inside this bin?  (it ends where count reaches k or mass reaches p)
        if (hcnt[bb] > 0 && (c + hcnt[bb] >= k_limit || m + hmass[bb] >= p_limit || bb == 0)) {
          bsel = bb;
          break;
        }
        c += hcnt[bb];
        m += hmass[bb];
        bsel = bb;
      }
      sh_bin = bsel;
      sh_cnt_above = c;
      sh_mass_above = m;
    }
    __syncthreads();
    prefix |= (uint32_t)sh_bin << shift;
    mask |= 0xffu << shift;
    cnt_above = sh_cnt_above;
    mass_above = sh_mass_above;
    __syncthreads();
  }
  // kept: key > prefix, plus threshold ties in id order while count < k and mass before < p
  // pass A: total kept mass ; pass B: walk to u * kept
  const float u = uniform ? uniform[b] : 0.5f;
  unsigned long long kept_total = 0, target = 0;
  for (int pass = 0; pass < 2; ++pass) {
    unsigned long long run = 0;          // kept mass so far (id order)
    int eq_cnt = 0;                      // threshold ties kept so far
    unsigned long long eq_mass = 0;
    int found = -1;
    for (int c0 = 0; c0 < v; c0 += 1024) {
      const int i = c0 + tid;
      float x = -INFINITY;
      uint32_t key = 0;
      if (i < v) x = val(i), key = okey(x);
      const unsigned long long pm = i < v ? fx(expf((x - mx) * inv_t)) : 0ull;
      const int eq = i < v && key == prefix;
      unsigned long long eqm_tot, dummy;
      const unsigned long long eqm_before = eq_mass + block_scan_u64(eq ? pm : 0ull, wt, eqm_tot);
      unsigned long long eqc_tot;
      const int eqc_before = eq_cnt + (int)block_scan_u64(eq ? 1ull : 0ull, wt, eqc_tot);
      const bool keep = i < v && (key > prefix || (eq && cnt_above + eqc_before < k_limit &&
                                                   mass_above + eqm_before < p_limit));
      const unsigned long long before = run + block_scan_u64(keep ? pm : 0ull, wt, dummy);
      if (pass == 1 && keep && before + pm > target && before <= target) found = i;
      run += dummy;
      eq_cnt += (int)eqc_tot;
      eq_mass += eqm_tot;
      if (pass == 1) {
        __syncthreads();
        if (found >= 0) si[1] = found;
        __syncthreads();
      }
    }
    if (pass == 0) {
      kept_total = run;
      double tt = (double)u * (double)kept_total;
      target = (unsigned long long)tt;
      if (target >= kept_total && kept_total > 0) target = kept_total - 1;
      if (tid == 0) si[1] = amax;
      __syncthreads();
    }
  }
  __syncthreads();
  if (tid == 0) out[b] = si[1];
}

}  // namespace

DSV4_API int dsv4_sample(const float* logits, int rows, int v, const float* temperature, const int* top_k,
                         const float* top_p, const float* uniform, const int* mask_ids, int n_mask, long long* out,
                         cudaStream_t st) {
  if (rows <= 0) return 0;
  dsv4_launch(sample_kernel, rows, 1024, 0, st, logits, v, temperature, top_k, top_p, uniform, mask_ids, n_mask, out);
  return (int)cudaGetLastError();
}
