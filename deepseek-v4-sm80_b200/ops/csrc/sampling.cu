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
// p * 2^40 truncated.  Multiplying a float by a power of two is exact, so the single-precision product equals the
// double-precision one the oracle computes; the FP64 pipe (slow on this part) stays out of the per-element path.
__device__ __forceinline__ unsigned long long fx(float p) { return __float2ull_rz(p * 1099511627776.0f); }

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
    // Histogram of the candidates' next key byte.  The top bytes of nearly all logits agree, so per-element atomics
    // would serialise on a handful of addresses: a warp whose active lanes all hit one bin adds once (the masses are
    // fixed point, so any order gives the same sums).
    for (int i0 = 0; i0 < v; i0 += 1024) {
      const int i = i0 + tid;
      bool act = false;
      uint32_t bin = 0;
      unsigned long long m = 0;
      if (i < v) {
        const float x = val(i);
        const uint32_t key = okey(x);
        if ((key & mask) == prefix) {
          act = true;
          bin = (key >> shift) & 0xff;
          m = fx(expf((x - mx) * inv_t));
        }
      }
      // one pair of atomics per distinct bin of the warp: 64-bit shared atomics under same-address contention are
      // what made the first version of this loop take milliseconds
      unsigned todo = __ballot_sync(0xffffffffu, act);
      while (todo) {  // `todo` is warp-uniform
        const int leader = __ffs(todo) - 1;
        const uint32_t bin0 = __shfl_sync(0xffffffffu, bin, leader);
        const bool mine = act && bin == bin0;
        const unsigned grp = __ballot_sync(0xffffffffu, mine);
        unsigned long long sm = mine ? m : 0ull;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sm += __shfl_xor_sync(0xffffffffu, sm, o);
        if (lane == leader) {
          atomicAdd(&hcnt[bin0], __popc(grp));
          atomicAdd(&hmass[bin0], sm);
        }
        todo &= ~grp;
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
  // kept: key > prefix, plus threshold ties in id order while count < k and mass before < p.
  // Every thread owns a contiguous range of ids, so "in id order" needs three block scans in total (ties before the
  // thread, tie mass before it, kept mass before it) and sequential walks inside the thread's own range.
  const float u = uniform ? uniform[b] : 0.5f;
  const int per = (v + 1023) / 1024;
  const int i_lo = min(tid * per, v), i_hi = min(i_lo + per, v);
  unsigned long long my_eq_mass = 0;
  int my_eq_cnt = 0;
  for (int i = i_lo; i < i_hi; ++i) {
    const float x = val(i);
    if (okey(x) == prefix) ++my_eq_cnt, my_eq_mass += fx(expf((x - mx) * inv_t));
  }
  unsigned long long tot;
  const int eqc_before = (int)block_scan_u64((unsigned long long)my_eq_cnt, wt, tot);
  const unsigned long long eqm_before = block_scan_u64(my_eq_mass, wt, tot);
  auto walk = [&](unsigned long long start, unsigned long long target, bool find) -> unsigned long long {
    // returns the kept mass of this thread's range, or (find) the id at which the running kept mass passes target
    unsigned long long run = start, em = eqm_before;
    int ec = eqc_before;
    for (int i = i_lo; i < i_hi; ++i) {
      const float x = val(i);
      const uint32_t key = okey(x);
      const unsigned long long pm = fx(expf((x - mx) * inv_t));
      const bool eq = key == prefix;
      const bool keep = key > prefix || (eq && cnt_above + ec < k_limit && mass_above + em < p_limit);
      if (eq) ++ec, em += pm;
      if (keep) {
        if (find && run + pm > target && run <= target) return (unsigned long long)i;
        run += pm;
      }
    }
    return find ? ~0ull : run - start;
  };
  const unsigned long long my_kept = walk(0ull, 0ull, false);
  unsigned long long kept_total;
  const unsigned long long kept_before = block_scan_u64(my_kept, wt, kept_total);
  unsigned long long target = (unsigned long long)((double)u * (double)kept_total);
  if (target >= kept_total && kept_total > 0) target = kept_total - 1;
  if (tid == 0) si[1] = amax;  // fallback (empty kept set cannot happen: the maximum is always kept)
  __syncthreads();
  if (my_kept > 0 && target >= kept_before && target < kept_before + my_kept) {
    const unsigned long long id = walk(kept_before, target, true);
    if (id != ~0ull) si[1] = (int)id;
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
