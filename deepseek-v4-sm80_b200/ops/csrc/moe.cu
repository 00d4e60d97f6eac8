// Routed-expert path of the MoE: router post-processing, route planning, token permutation, a persistent
// tcgen05 grouped GEMM over packed-FP4 expert weights (W4A16), and the final per-token reduction.
//
// The grouped GEMM computes, per (expert, 128 weight rows, <=NT routes) tile,  D[row, route] = W[row, :] . X[route, :]
// ("swap-AB": the weight rows sit on the 128 TMEM lanes, routes are the UMMA N dimension, so an expert with a
// handful of routes costs an N=16..NT instruction instead of a padded M=128 one).  Warp roles per CTA:
//   warp 0      TMA producer: packed FP4 weight k-stages (128 rows x 128 B, 128-byte swizzle) and, per 64-wide
//               k sub-tile, the bf16 route rows (already permuted into expert order) straight into the UMMA operand
//   warp 1      tcgen05.mma issuer (kind::f16), accumulators double-buffered in TMEM across tiles
//   warps 2-5   epilogue: tcgen05.ld, then SwiGLU-with-clamp (GEMM1) or route-weight scaling (GEMM2)
//   warps 6-13  operand builders: E2M1 nibbles -> bf16 * 2^(e8m0-127) written as the K-major 128B-swizzled
//               UMMA A tile (generic-proxy stores + fence.proxy.async)
// Numerics match the reference's Marlin path (python/minisgl/kernel/marlin_wna16.py:288-356): bf16 activations,
// exact FP4 dequantisation, fp32 accumulation, GEMM1 output rounded to bf16 before the fp32 SwiGLU, GEMM2
// output rounded to bf16 and multiplied by the bf16 route weight, routes summed afterwards.
#include "comm.cuh"

namespace {

constexpr int kRowsTile = 128;
constexpr int kPStages = 3;     // packed-weight stages (256 K elements each)
constexpr int kOBufs = 2;       // bf16 operand buffers (64 K elements each)
constexpr int kBuilders = 256;  // builder threads
constexpr int kThreads = 64 + 128 + kBuilders;

struct PlanHeader {
  int num_tiles;
  int num_routes_local;
  int pad0, pad1;
};

// ------------------------------------------------------------------ router post-processing
// scores fp32 [T,E] -> p = sqrt(softplus) | sigmoid ; select top-k of p + bias (ties: lower id) or the hash
// table row; w = p[idx] / (sum + 1e-8) * scaling.  Rows >= num_valid get (-1, 0).
__global__ void moe_topk_kernel(const float* __restrict__ scores, const float* __restrict__ bias,
                                const int* __restrict__ tid2eid, const int* __restrict__ token_ids,
                                const int* __restrict__ num_valid, int* __restrict__ idx, float* __restrict__ wts,
                                int t_rows, int e, int k, float scaling, int scoring) {
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (row >= t_rows) return;
  if (num_valid && row >= *num_valid) {
    if (lane < k) idx[row * k + lane] = -1, wts[row * k + lane] = 0.f;
    return;
  }
  constexpr int MAXPER = 16;  // e <= 512
  float p[MAXPER], sel[MAXPER];
  const int per = (e + 31) / 32;
  float smax = -INFINITY;
  if (scoring == 2) {
    for (int i = 0; i < per; ++i) {
      const int j = lane + i * 32;
      if (j < e) smax = fmaxf(smax, scores[(size_t)row * e + j]);
    }
    smax = warp_max(smax);
  }
  float ssum = 0.f;
#pragma unroll
  for (int i = 0; i < MAXPER; ++i) {
    const int j = lane + i * 32;
    p[i] = 0.f;
    sel[i] = -INFINITY;
    if (i < per && j < e) {
      const float s = scores[(size_t)row * e + j];
      float v;
      if (scoring == 0) {
        const float sp = s > 20.f ? s : log1pf(expf(s));
        v = sqrtf(sp);
      } else if (scoring == 1) {
        v = 1.f / (1.f + expf(-s));
      } else {
        v = expf(s - smax);
        ssum += v;
      }
      p[i] = v;
    }
  }
  if (scoring == 2) {
    ssum = warp_sum(ssum);
#pragma unroll
    for (int i = 0; i < MAXPER; ++i) p[i] /= ssum;
  }
#pragma unroll
  for (int i = 0; i < MAXPER; ++i) {
    const int j = lane + i * 32;
    if (i < per && j < e) sel[i] = p[i] + (bias ? bias[j] : 0.f);
  }
  float wsum = 0.f;
  float myw = 0.f;
  int myi = -1;
  for (int r = 0; r < k; ++r) {
    int bi;
    float bp;
    if (tid2eid) {
      bi = tid2eid[(size_t)token_ids[row] * k + r];
    } else {
      float bv = -INFINITY;
      bi = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < MAXPER; ++i) {
        const int j = lane + i * 32;
        if (sel[i] > bv || (sel[i] == bv && j < bi && sel[i] > -INFINITY)) bv = sel[i], bi = j;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) bv = ov, bi = oi;
      }
    }
    // owner lane publishes p[bi] and retires the entry
    float pv = 0.f;
#pragma unroll
    for (int i = 0; i < MAXPER; ++i) {
      const int j = lane + i * 32;
      if (j == bi) {
        pv = p[i];
        sel[i] = -INFINITY;
      }
    }
    bp = __shfl_sync(0xffffffffu, pv, bi & 31);
    wsum += bp;
    if (lane == r) myw = bp, myi = bi;
  }
  if (lane < k) {
    idx[row * k + lane] = myi;
    wts[row * k + lane] = myw / (wsum + 1e-8f) * scaling;
  }
}

// ------------------------------------------------------------------ route planning (one CTA)
// Local routes (expert in [base, base+e_local)) are grouped by expert; order inside a group is arbitrary
// (every route row is computed independently and lands in its own output row, so results do not depend on it).
__global__ void __launch_bounds__(1024) moe_plan_kernel(const int* __restrict__ idx, const float* __restrict__ wts,
                                                        int routes, int e_local, int base, int nt,
                                                        PlanHeader* __restrict__ hdr, int* __restrict__ tiles,
                                                        int* __restrict__ sorted_route, int* __restrict__ route_pos,
                                                        float* __restrict__ sorted_w) {
  extern __shared__ int sm[];
  int* cnt = sm;                 // [e_local]
  int* off = sm + e_local;       // [e_local + 1]
  int* cur = off + e_local + 1;  // [e_local]
  int* toff = cur + e_local;     // [e_local + 1]
  for (int i = threadIdx.x; i < e_local; i += blockDim.x) cnt[i] = 0;
  __syncthreads();
  for (int r = threadIdx.x; r < routes; r += blockDim.x) {
    const int e = idx[r] - base;
    if (idx[r] >= 0 && e >= 0 && e < e_local) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int a = 0, ta = 0;
    for (int i = 0; i < e_local; ++i) {
      off[i] = a;
      toff[i] = ta;
      a += cnt[i];
      ta += (cnt[i] + nt - 1) / nt;
    }
    off[e_local] = a;
    toff[e_local] = ta;
    hdr->num_tiles = ta;
    hdr->num_routes_local = a;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < e_local; i += blockDim.x) {
    cur[i] = 0;
    const int n = cnt[i];
    for (int c = 0, ti = toff[i]; c < n; c += nt, ++ti) {
      tiles[ti * 3 + 0] = i;
      tiles[ti * 3 + 1] = off[i] + c;
      tiles[ti * 3 + 2] = min(nt, n - c);
    }
  }
  __syncthreads();
  for (int r = threadIdx.x; r < routes; r += blockDim.x) {
    const int e = idx[r] - base;
    if (idx[r] >= 0 && e >= 0 && e < e_local) {
      const int pos = off[e] + atomicAdd(&cur[e], 1);
      sorted_route[pos] = r;
      sorted_w[pos] = wts[r];
      route_pos[r] = pos;
    } else {
      route_pos[r] = -1;
    }
  }
}

// xs[pos] = x[route / topk]
__global__ void moe_permute_kernel(const uint4* __restrict__ x, uint4* __restrict__ xs,
                                   const int* __restrict__ sorted_route, const PlanHeader* __restrict__ hdr, int topk,
                                   int h8) {
  const int pos = blockIdx.x;
  if (pos >= hdr->num_routes_local) return;
  const int tok = sorted_route[pos] / topk;
  for (int i = threadIdx.x; i < h8; i += blockDim.x) xs[(size_t)pos * h8 + i] = x[(size_t)tok * h8 + i];
}

// ------------------------------------------------------------------ FP4 -> bf16 operand builder
// 8 packed nibbles (one 32-bit word = elements 8c..8c+7, low nibble first) -> 8 bf16 scaled by 2^(sc-127).
// A nibble s.e1e0.m placed at bf16 bits [8:6] (sign at 15) reads as value * 2^-126, so one packed multiply by
// 2^(sc-1) yields the exact dequantised weight (sc is the e8m0 byte; sc <= 128 is required and checked on load).
__device__ __forceinline__ uint4 dequant8(uint32_t w, uint32_t mul2) {
  uint32_t r[4];
  const uint32_t lo = w & 0x0F0F0F0Fu, hi = (w >> 4) & 0x0F0F0F0Fu;
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    // byte p of lo -> low half, byte p of hi -> high half
    const uint32_t x = __byte_perm(lo, hi, 0x4040 + p + ((4 + p) << 8)) & 0x000F000Fu;  // [lo.bp, 0, hi.bp, 0]
    const uint32_t bits = ((x & 0x00070007u) << 6) | ((x & 0x00080008u) << 12);
    __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&bits);
    const __nv_bfloat162 m = *reinterpret_cast<const __nv_bfloat162*>(&mul2);
    v = __hmul2(v, m);
    r[p] = *reinterpret_cast<uint32_t*>(&v);
  }
  return make_uint4(r[0], r[1], r[2], r[3]);
}
__device__ __forceinline__ uint32_t scale_mul2(uint32_t sc) {
  // bf16 2^(sc-1): exponent field sc+126 (sc in [1,128]); sc == 0 -> 0
  const uint32_t f = sc == 0 ? 0u : min(sc + 126u, 254u);
  const uint32_t h = f << 7;
  return h | (h << 16);
}

template <int MODE, int NT>
struct MoeSmem {
  static constexpr int kMats = MODE == 1 ? 2 : 1;
  static constexpr int kPackedBytes = kMats * kRowsTile * 128;  // per packed stage
  static constexpr int kABytes = kRowsTile * 128;               // one bf16 operand sub-tile
  static constexpr int kBBytes = NT * 128;
  static constexpr int kOBytes = kMats * kABytes + kBBytes;
  static constexpr int kTotal = kPStages * kPackedBytes + kOBufs * kOBytes + 1024 + 512;
};

// MODE 1: D_gate, D_up -> act[pos, j] = bf16(silu(min(g,L)) * clamp(u,+-L)), weights w13 [E, 2I, K/2].
// MODE 2: D -> out[route, h] = bf16(bf16(acc) * bf16(w_route)), weights w2 [E, H, K/2].
template <int MODE, int NT>
__global__ void __launch_bounds__(kThreads, 1)
moe_gemm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                const uint8_t* __restrict__ scales, const PlanHeader* __restrict__ hdr, const int* __restrict__ tiles,
                const int* __restrict__ sorted_route, const float* __restrict__ sorted_w,
                __nv_bfloat16* __restrict__ out, int K, int rows_per_expert /*I (mode1) or H (mode2)*/,
                int ld_out, float limit) {
  using S = MoeSmem<MODE, NT>;
  constexpr int kMats = S::kMats;
  constexpr uint32_t kTmemCols = 2 * kMats * NT < 32 ? 32 : 2 * kMats * NT;  // double-buffered accumulators
  constexpr uint32_t kIdesc = umma_idesc(128, NT, 1, 1);
  extern __shared__ uint8_t moe_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(moe_smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* packed = smem;
  uint8_t* obuf = smem + kPStages * S::kPackedBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(obuf + kOBufs * S::kOBytes);
  uint64_t* pfull = bars;               // [kPStages]
  uint64_t* pempty = pfull + kPStages;  // [kPStages]
  uint64_t* ofull = pempty + kPStages;  // [kOBufs]
  uint64_t* oempty = ofull + kOBufs;    // [kOBufs]
  uint64_t* tfull = oempty + kOBufs;    // [2]
  uint64_t* tempty = tfull + 2;         // [2]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row_tiles = rows_per_expert / kRowsTile;
  const int kstages = K / 256;
  const int scale_ld = K / 32;  // scale bytes per weight row

  if (threadIdx.x == 0) {
    for (int i = 0; i < kPStages; ++i) mbar_init(&pfull[i], 1), mbar_init(&pempty[i], kBuilders);
    for (int i = 0; i < kOBufs; ++i) mbar_init(&ofull[i], kBuilders + 1), mbar_init(&oempty[i], 1);
    for (int i = 0; i < 2; ++i) mbar_init(&tfull[i], 1), mbar_init(&tempty[i], 128);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const int total_work = hdr->num_tiles * row_tiles;

  if (warp == 0) {
    if (lane == 0) {
      int ps = 0, ob = 0;  // running packed-stage / operand-buffer counters
      for (int wk = blockIdx.x; wk < total_work; wk += gridDim.x) {
        const int ct = wk / row_tiles, rt = wk % row_tiles;
        const int e = tiles[ct * 3], tok0 = tiles[ct * 3 + 1];
        const int wrow = e * (MODE == 1 ? 2 * rows_per_expert : rows_per_expert) + rt * kRowsTile;
        bool ok = true;
        for (int ks = 0; ks < kstages && ok; ++ks, ++ps) {
          const int s = ps % kPStages;
          if (!mbar_wait(&pempty[s], ((ps / kPStages) & 1) ^ 1, abort_flag, 11)) { ok = false; break; }
          mbar_expect_tx(&pfull[s], S::kPackedBytes);
          uint8_t* dst = packed + s * S::kPackedBytes;
          tma_load_2d(dst, &tmW, &pfull[s], ks * 128, wrow);
          if (MODE == 1) tma_load_2d(dst + kRowsTile * 128, &tmW, &pfull[s], ks * 128, wrow + rows_per_expert);
          for (int q = 0; q < 4; ++q, ++ob) {
            const int b = ob % kOBufs;
            if (!mbar_wait(&oempty[b], ((ob / kOBufs) & 1) ^ 1, abort_flag, 12)) { ok = false; break; }
            mbar_expect_tx(&ofull[b], S::kBBytes);
            tma_load_2d(obuf + b * S::kOBytes + kMats * S::kABytes, &tmX, &ofull[b], ks * 256 + q * 64, tok0);
          }
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int ob = 0, it = 0;
      for (int wk = blockIdx.x; wk < total_work; wk += gridDim.x, ++it) {
        const int acc = it & 1;
        if (!mbar_wait(&tempty[acc], ((it >> 1) & 1) ^ 1, abort_flag, 13)) break;
        tc_fence_after();
        const uint32_t d0 = tmem_base + acc * kMats * NT;
        bool ok = true;
        for (int sub = 0; sub < kstages * 4; ++sub, ++ob) {
          const int b = ob % kOBufs;
          if (!mbar_wait(&ofull[b], (ob / kOBufs) & 1, abort_flag, 14)) { ok = false; break; }
          tc_fence_after();
          const uint8_t* a = obuf + b * S::kOBytes;
          const uint8_t* bt = a + kMats * S::kABytes;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t bd = umma_desc_k128(bt, k * 32);
            umma_f16(d0, umma_desc_k128(a, k * 32), bd, kIdesc, (sub > 0 || k > 0));
            if (MODE == 1) umma_f16(d0 + NT, umma_desc_k128(a + S::kABytes, k * 32), bd, kIdesc, (sub > 0 || k > 0));
          }
          umma_commit(&oempty[b]);
        }
        if (!ok) break;
        umma_commit(&tfull[acc]);
      }
    }
  } else if (warp < 6) {
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    int it = 0;
    for (int wk = blockIdx.x; wk < total_work; wk += gridDim.x, ++it) {
      const int acc = it & 1;
      const int ct = wk / row_tiles, rt = wk % row_tiles;
      const int tok0 = tiles[ct * 3 + 1], ntok = tiles[ct * 3 + 2];
      if (!mbar_wait(&tfull[acc], (it >> 1) & 1, abort_flag, 15)) break;
      tc_fence_after();
      const uint32_t d0 = lane_addr + acc * kMats * NT;
      const int orow = rt * kRowsTile + r;  // intermediate index (mode 1) / hidden index (mode 2)
#pragma unroll 1
      for (int c0 = 0; c0 < NT; c0 += 32) {
        if (c0 >= ntok) break;
        uint32_t g[32];
        tmem_ld_32x32(d0 + c0, g);
        if (MODE == 1) {
          uint32_t u[32];
          tmem_ld_32x32(d0 + NT + c0, u);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            if (c0 + c < ntok) {
              float gv = bf2f(f2bf(__uint_as_float(g[c]))), uv = bf2f(f2bf(__uint_as_float(u[c])));
              if (limit > 0.f) {
                gv = fminf(gv, limit);
                uv = fminf(fmaxf(uv, -limit), limit);
              }
              const float a = gv / (1.f + expf(-gv)) * uv;
              out[(size_t)(tok0 + c0 + c) * ld_out + orow] = f2bf(a);
            }
          }
        } else {
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            if (c0 + c < ntok) {
              const int pos = tok0 + c0 + c;
              const __nv_bfloat16 y = f2bf(__uint_as_float(g[c]));
              const __nv_bfloat16 wv = f2bf(sorted_w[pos]);
              out[(size_t)sorted_route[pos] * ld_out + orow] = __hmul(y, wv);
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&tempty[acc]);
    }
  } else {
    // builders: thread b -> weight row (b % 128); MODE 1: matrix b / 128, all 4 sub-tiles of a stage;
    // MODE 2: sub-tiles {2*(b/128), 2*(b/128)+1}
    const int bt = threadIdx.x - 192;
    const int r = bt & 127, half = bt >> 7;
    int ps = 0, ob = 0;
    for (int wk = blockIdx.x; wk < total_work; wk += gridDim.x) {
      const int ct = wk / row_tiles, rt = wk % row_tiles;
      const int e = tiles[ct * 3];
      const size_t wrow = (size_t)e * (MODE == 1 ? 2 * rows_per_expert : rows_per_expert) + rt * kRowsTile + r +
                          (MODE == 1 ? half * rows_per_expert : 0);
      const uint8_t* srow = scales + wrow * scale_ld;
      bool ok = true;
      for (int ks = 0; ks < kstages && ok; ++ks, ++ps) {
        const int s = ps % kPStages;
        const uint2 scv = *reinterpret_cast<const uint2*>(srow + ks * 8);  // 8 scale bytes: 2 per sub-tile
        if (!mbar_wait(&pfull[s], (ps / kPStages) & 1, abort_flag, 16)) { ok = false; break; }
        const uint8_t* prow = packed + s * S::kPackedBytes + (MODE == 1 ? half * kRowsTile * 128 : 0) + r * 128;
        for (int q = 0; q < 4; ++q, ++ob) {
          const int b = ob % kOBufs;
          if (!mbar_wait(&oempty[b], ((ob / kOBufs) & 1) ^ 1, abort_flag, 17)) { ok = false; break; }
          if (MODE == 1 || (q >> 1) == half) {
            const uint32_t sw = q < 2 ? scv.x : scv.y;
            const uint32_t m0 = scale_mul2((sw >> ((q & 1) * 16)) & 0xff);
            const uint32_t m1 = scale_mul2((sw >> ((q & 1) * 16 + 8)) & 0xff);
            // packed sub-tile q = bytes [32q, 32q+32) of the 128-byte row = 16B chunks 2q, 2q+1 (swizzled by row)
            const uint4 p0 = *reinterpret_cast<const uint4*>(prow + (((2 * q) ^ (r & 7)) << 4));
            const uint4 p1 = *reinterpret_cast<const uint4*>(prow + (((2 * q + 1) ^ (r & 7)) << 4));
            uint8_t* arow = obuf + b * S::kOBytes + (MODE == 1 ? half * S::kABytes : 0) + r * 128;
            const uint32_t w[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
            for (int c = 0; c < 8; ++c)
              *reinterpret_cast<uint4*>(arow + ((c ^ (r & 7)) << 4)) = dequant8(w[c], c < 4 ? m0 : m1);
          }
          fence_proxy_async_smem();
          mbar_arrive(&ofull[b]);
        }
        if (ok) mbar_arrive(&pempty[s]);
      }
      if (!ok) break;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

// out[t] = bf16( float(bf16(sum_k local route rows)) + float(shared[t]) ); rows >= num_valid -> 0
__global__ void moe_finalize_kernel(const __nv_bfloat16* __restrict__ yr, const int* __restrict__ route_pos,
                                    const __nv_bfloat16* __restrict__ shared, __nv_bfloat16* __restrict__ out,
                                    const int* __restrict__ num_valid, int topk, int h) {
  const int t = blockIdx.x;
  const bool valid = !num_valid || t < *num_valid;
  for (int i = threadIdx.x * 8; i < h; i += blockDim.x * 8) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    uint4 o = make_uint4(0, 0, 0, 0);
    if (valid) {
      for (int k = 0; k < topk; ++k) {
        if (route_pos[t * topk + k] < 0) continue;
        const uint4 u = *reinterpret_cast<const uint4*>(yr + ((size_t)t * topk + k) * h + i);
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(p[j]);
          acc[2 * j] += f.x, acc[2 * j + 1] += f.y;
        }
      }
      uint4 su = make_uint4(0, 0, 0, 0);
      if (shared) su = *reinterpret_cast<const uint4*>(shared + (size_t)t * h + i);
      const __nv_bfloat162* sp = reinterpret_cast<const __nv_bfloat162*>(&su);
      __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 r2 = __bfloat1622float2(__floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]));
        const float2 s2 = __bfloat1622float2(sp[j]);
        po[j] = __floats2bfloat162_rn(r2.x + s2.x, r2.y + s2.y);
      }
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * h + i) = o;
  }
}

// Fused combine: the per-token sum of the local routes (+ the shared expert) is this rank's partial of the layer
// output; it goes to the symmetric buffer and is reduced across ranks in the same kernel (protocol in comm.cuh).
__global__ void __launch_bounds__(256) moe_finalize_ar_kernel(const __nv_bfloat16* __restrict__ yr,
                                                              const int* __restrict__ route_pos,
                                                              const __nv_bfloat16* __restrict__ shared,
                                                              __nv_bfloat16* __restrict__ out,
                                                              const int* __restrict__ num_valid, int topk, int h,
                                                              int t_rows, const CommCtx comm) {
  __shared__ int ok;
  const uint32_t epoch = comm_epoch(comm);
  const int parity = epoch & 1;
  __nv_bfloat16* mine = comm_data(comm, comm.rank, parity);
  const int nv = num_valid ? *num_valid : t_rows;
  for (int t = blockIdx.x; t < t_rows; t += gridDim.x) {
    const bool valid = t < nv;
    for (int i = threadIdx.x * 8; i < h; i += blockDim.x * 8) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      uint4 o = make_uint4(0, 0, 0, 0);
      if (valid) {
        for (int k = 0; k < topk; ++k) {
          if (route_pos[t * topk + k] < 0) continue;
          const uint4 u = *reinterpret_cast<const uint4*>(yr + ((size_t)t * topk + k) * h + i);
          const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(p[j]);
            acc[2 * j] += f.x, acc[2 * j + 1] += f.y;
          }
        }
        const uint4 su = *reinterpret_cast<const uint4*>(shared + (size_t)t * h + i);
        const __nv_bfloat162* sp = reinterpret_cast<const __nv_bfloat162*>(&su);
        __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 r2 = __bfloat1622float2(__floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]));
          const float2 s2 = __bfloat1622float2(sp[j]);
          po[j] = __floats2bfloat162_rn(r2.x + s2.x, r2.y + s2.y);
        }
      }
      *reinterpret_cast<uint4*>(mine + (size_t)t * h + i) = o;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    comm_publish(comm, blockIdx.x, epoch);
    ok = comm_wait(comm, blockIdx.x, epoch) ? 1 : 0;
  }
  __syncthreads();
  if (ok) {
    for (int t = blockIdx.x; t < t_rows; t += gridDim.x)
      for (int i = threadIdx.x * 8; i < h; i += blockDim.x * 8)
        *reinterpret_cast<uint4*>(out + (size_t)t * h + i) = comm_reduce16(comm, parity, (size_t)t * h + i);
  }
  __syncthreads();
  if (threadIdx.x == 0) comm_finish(comm, gridDim.x);
}

template <int MODE, int NT>
int launch_moe_gemm(const void* w, const uint8_t* scales, const void* x, int x_rows, const PlanHeader* hdr,
                    const int* tiles, const int* sorted_route, const float* sorted_w, void* out, int e_local, int K,
                    int rows_per_expert, int ld_out, float limit, int num_sms, cudaStream_t st) {
  using S = MoeSmem<MODE, NT>;
  CUtensorMap tmW, tmX;
  const uint64_t wrows = (uint64_t)e_local * (MODE == 1 ? 2 : 1) * rows_per_expert;
  if (dsv4_make_tmap_2d(&tmW, w, 0, (uint64_t)K / 2, wrows, (uint64_t)K / 2, 128, kRowsTile, 3)) return 201;
  if (dsv4_make_tmap_2d(&tmX, x, 1, (uint64_t)K, (uint64_t)x_rows, (uint64_t)K * 2, 64, NT, 3)) return 202;
  auto kern = moe_gemm_kernel<MODE, NT>;
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal) != cudaSuccess) return 203;
    set = true;
  }
  kern<<<num_sms, kThreads, S::kTotal, st>>>(tmW, tmX, scales, hdr, tiles, sorted_route, sorted_w, (__nv_bfloat16*)out,
                                            K, rows_per_expert, ld_out, limit);
  return (int)cudaGetLastError();
}

}  // namespace

DSV4_API int dsv4_moe_topk(const float* scores, const float* bias, const int* tid2eid, const int* token_ids,
                           const int* num_valid, int* idx, float* wts, int t, int e, int k, float scaling, int scoring,
                           cudaStream_t st) {
  if (t <= 0) return 0;
  if (e > 512 || k > 32) return 210;
  moe_topk_kernel<<<(t * 32 + 255) / 256, 256, 0, st>>>(scores, bias, tid2eid, token_ids, num_valid, idx, wts, t, e, k,
                                                       scaling, scoring);
  return (int)cudaGetLastError();
}

// plan buffer layout (ints): [hdr(4)] [tiles 3*max_tiles] [sorted_route R] [route_pos R] [sorted_w R (float)]
DSV4_API int dsv4_moe_plan(const int* idx, const float* wts, int routes, int e_local, int base, int nt, int* plan,
                           int max_tiles, cudaStream_t st) {
  PlanHeader* hdr = reinterpret_cast<PlanHeader*>(plan);
  int* tiles = plan + 4;
  int* sorted_route = tiles + 3 * max_tiles;
  int* route_pos = sorted_route + routes;
  float* sorted_w = reinterpret_cast<float*>(route_pos + routes);
  const int smem = (4 * e_local + 2) * sizeof(int);
  moe_plan_kernel<<<1, 1024, smem, st>>>(idx, wts, routes, e_local, base, nt, hdr, tiles, sorted_route, route_pos,
                                         sorted_w);
  return (int)cudaGetLastError();
}

DSV4_API int dsv4_moe_permute(const void* x, void* xs, const int* plan, int routes, int max_tiles, int topk, int h,
                              cudaStream_t st) {
  if (routes <= 0) return 0;
  const PlanHeader* hdr = reinterpret_cast<const PlanHeader*>(plan);
  const int* sorted_route = plan + 4 + 3 * max_tiles;
  moe_permute_kernel<<<routes, 128, 0, st>>>((const uint4*)x, (uint4*)xs, sorted_route, hdr, topk, h / 8);
  return (int)cudaGetLastError();
}

// mode 1: x = permuted tokens [routes, K=H] -> out = act [routes, I];  mode 2: x = act [routes, K=I] -> out = route rows
DSV4_API int dsv4_moe_gemm(int mode, int nt, const void* w, const void* scales, const void* x, int x_rows,
                           const int* plan, int routes, int max_tiles, void* out, int e_local, int K,
                           int rows_per_expert, int ld_out, float limit, int num_sms, cudaStream_t st) {
  if (K % 256 || rows_per_expert % kRowsTile) return 220;
  const PlanHeader* hdr = reinterpret_cast<const PlanHeader*>(plan);
  const int* tiles = plan + 4;
  const int* sorted_route = tiles + 3 * max_tiles;
  const float* sorted_w = reinterpret_cast<const float*>(sorted_route + 2 * routes);
  const uint8_t* sc = (const uint8_t*)scales;
#define MOE_LAUNCH(M, N)                                                                                        \
  return launch_moe_gemm<M, N>(w, sc, x, x_rows, hdr, tiles, sorted_route, sorted_w, out, e_local, K,           \
                               rows_per_expert, ld_out, limit, num_sms, st)
  if (mode == 1 && nt == 32) MOE_LAUNCH(1, 32);
  if (mode == 1 && nt == 128) MOE_LAUNCH(1, 128);
  if (mode == 2 && nt == 32) MOE_LAUNCH(2, 32);
  if (mode == 2 && nt == 128) MOE_LAUNCH(2, 128);
#undef MOE_LAUNCH
  return 221;
}

DSV4_API int dsv4_moe_finalize(const void* yr, const int* plan, int routes, int max_tiles, const void* shared, void* out,
                               const int* num_valid, int t, int topk, int h, cudaStream_t st) {
  if (t <= 0) return 0;
  const int* route_pos = plan + 4 + 3 * max_tiles + routes;
  moe_finalize_kernel<<<t, 256, 0, st>>>((const __nv_bfloat16*)yr, route_pos, (const __nv_bfloat16*)shared,
                                         (__nv_bfloat16*)out, num_valid, topk, h);
  return (int)cudaGetLastError();
}

DSV4_API int dsv4_moe_finalize_allreduce(const void* yr, const int* plan, int routes, int max_tiles, const void* shared,
                                         void* out, const int* num_valid, int t, int topk, int h, const CommCtx* comm,
                                         cudaStream_t st) {
  if (t <= 0) return 0;
  if (h % 8 || (long long)t * h * 2 > comm->data_bytes) return 230;
  const int* route_pos = plan + 4 + 3 * max_tiles + routes;
  const int grid = t < 1024 ? t : 1024;
  moe_finalize_ar_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)yr, route_pos, (const __nv_bfloat16*)shared,
                                               (__nv_bfloat16*)out, num_valid, topk, h, t, *comm);
  return (int)cudaGetLastError();
}
