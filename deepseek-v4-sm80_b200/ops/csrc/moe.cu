// Routed-expert path of the MoE: router post-processing, route planning, token permutation, a persistent
// tcgen05 grouped GEMM over packed-FP4 expert weights (W4A16), and the final per-token reduction.
//
// The grouped GEMM computes, per (expert, 128 weight rows, <=NT routes) tile,  D[row, route] = W[row, :] . X[route, :]
// ("swap-AB": the weight rows sit on the 128 TMEM lanes, routes are the UMMA N dimension, so an expert with a
// handful of routes costs an N=16..NT instruction instead of a padded M=128 one).  Warp roles per CTA:
//   warp 0      TMA producer: packed FP4 weight k-stages (128 rows x 128 B, 128-byte swizzle) and, per 64-wide
//               k sub-tile, the fp16 route rows (already permuted into expert order) straight into the UMMA operand
//   warp 1      tcgen05.mma issuer (kind::f16), accumulators double-buffered in TMEM across tiles
//   warps 2-5   epilogue: tcgen05.ld, then SwiGLU-with-clamp (GEMM1) or route-weight scaling (GEMM2)
//   warps 6-21  operand builders: E2M1 nibbles -> fp16 * 2^(e8m0-127), stored with tcgen05.st as the UMMA A operand
//               in tensor memory (a dequantised tile never touches shared memory, whose bandwidth it would exhaust)
//   warp 22     TMA producer of the route rows
//   warp 23     second tcgen05.mma issuer
// Numerics match the reference's Marlin path (python/minisgl/kernel/marlin_wna16.py:288-356): bf16 activations
// (held as fp16 for the tensor core: exact for |x| in [2^-14, 65504]), exact FP4 dequantisation, fp32 accumulation, GEMM1 output rounded to bf16 before the fp32 SwiGLU, GEMM2
// output rounded to bf16 and multiplied by the bf16 route weight, routes summed afterwards.
#include "comm.cuh"
#include "hc_post.cuh"

namespace {

constexpr int kRowsTile = 128;
constexpr int kBuilders = 512;  // builder threads (two teams of 256)
constexpr int kThreads = 64 + 128 + kBuilders + 64;  // + the route-row producer warp and the second MMA issuer

struct PlanHeader {
  int num_tiles;
  int num_routes_local;
  int pad0, pad1;
};

// ------------------------------------------------------------------ router post-processing
// scores fp32 [n_part][T,E] (split-K partial products, summed here) -> p = sqrt(softplus) | sigmoid ; select top-k of p + bias (ties: lower id) or the hash
// table row; w = p[idx] / (sum + 1e-8) * scaling.  Rows >= num_valid get (-1, 0).
__global__ void moe_topk_kernel(const float* __restrict__ scores, const float* __restrict__ bias,
                                const int* __restrict__ tid2eid, const int* __restrict__ token_ids,
                                const int* __restrict__ num_valid, int* __restrict__ idx, float* __restrict__ wts,
                                int t_rows, int e, int k, float scaling, int scoring, int n_part,
                                long long part_stride) {
  pdl_entry();
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (row >= t_rows) return;  // the last CTA may hold a warp past the last token
  // scores come as n_part split-K partial products (spaced part_stride floats apart); they are added below in split
  // order, with the loads of all of a lane's experts in flight together
  if (num_valid && row >= *num_valid) {
    if (lane < k) idx[row * k + lane] = -1, wts[row * k + lane] = 0.f;
    return;
  }
  constexpr int MAXPER = 16;  // e <= 512
  float p[MAXPER], sel[MAXPER];
  const int per = (e + 31) / 32;
  float sc[MAXPER];
#pragma unroll
  for (int i = 0; i < MAXPER; ++i) sc[i] = 0.f;
  {
    const float* sp = scores + (size_t)row * e + lane;
#pragma unroll 2
    for (int q = 0; q < n_part; ++q) {
      float tmp[MAXPER];
#pragma unroll
      for (int i = 0; i < MAXPER; ++i)
        tmp[i] = (i < per && lane + i * 32 < e) ? __ldg(sp + (size_t)q * part_stride + i * 32) : 0.f;
#pragma unroll
      for (int i = 0; i < MAXPER; ++i) sc[i] += tmp[i];
    }
  }
  float smax = -INFINITY;
  if (scoring == 2) {
#pragma unroll
    for (int i = 0; i < MAXPER; ++i) {
      const int j = lane + i * 32;
      if (i < per && j < e) smax = fmaxf(smax, sc[i]);
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
      const float s = sc[i];
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
  pdl_entry();
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

// xs[pos] = fp16(x[route / topk]): the grouped GEMMs run fp16 x fp16 (FP4 weights convert to fp16 in one instruction).
// bf16 reaches far beyond fp16's range; an activation above 65 504 in magnitude saturates to the largest finite fp16
// instead of becoming infinity (normalised activations stay orders of magnitude below that).
__global__ void moe_permute_kernel(const uint4* __restrict__ x, uint4* __restrict__ xs,
                                   const int* __restrict__ sorted_route, const PlanHeader* __restrict__ hdr, int topk,
                                   int h8) {
  pdl_entry();
  const int pos = blockIdx.x;
  if (pos >= hdr->num_routes_local) return;
  const int tok = sorted_route[pos] / topk;
  for (int i = threadIdx.x; i < h8; i += blockDim.x) {
    const uint4 v = x[(size_t)tok * h8 + i];
    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
    uint4 o;
    __half2* hp = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __bfloat1622float2(b[j]);
      f.x = fminf(fmaxf(f.x, -65504.f), 65504.f);
      f.y = fminf(fmaxf(f.y, -65504.f), 65504.f);
      hp[j] = __float22half2_rn(f);
    }
    xs[(size_t)pos * h8 + i] = o;
  }
}

// ------------------------------------------------------------------ FP4 -> fp16 operand builder
// 8 packed nibbles (one 32-bit word = elements 8c..8c+7, low nibble first) -> 8 fp16 scaled by 2^(sc-127), where sc
// is the e8m0 scale byte of the 32-element group.  Scales in [103, 142] are exact; the loader rejects others.
__device__ __forceinline__ uint4 dequant8(uint32_t w, uint32_t mul2) {
  // Blackwell converts a byte holding two E2M1 values straight to an fp16 pair (low nibble -> low half); one packed
  // multiply applies the group scale.  Both steps are exact.
  uint32_t r0, r1, r2, r3;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\tmov.b32 {b0, b1, b2, b3}, %4;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\tcvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n\tcvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
      : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
      : "r"(w));
  const __half2 m = *reinterpret_cast<const __half2*>(&mul2);
  __half2 v0 = __hmul2(*reinterpret_cast<__half2*>(&r0), m), v1 = __hmul2(*reinterpret_cast<__half2*>(&r1), m);
  __half2 v2 = __hmul2(*reinterpret_cast<__half2*>(&r2), m), v3 = __hmul2(*reinterpret_cast<__half2*>(&r3), m);
  return make_uint4(*reinterpret_cast<uint32_t*>(&v0), *reinterpret_cast<uint32_t*>(&v1),
                    *reinterpret_cast<uint32_t*>(&v2), *reinterpret_cast<uint32_t*>(&v3));
}
// 32 packed nibbles (one 16-byte chunk) -> 32 fp16 in 16 registers, K order
__device__ __forceinline__ void dequant8x4(const uint4& p, uint32_t mul2, uint32_t (&v)[16]) {
  const uint4 a = dequant8(p.x, mul2), b = dequant8(p.y, mul2), c = dequant8(p.z, mul2), d = dequant8(p.w, mul2);
  v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w;
  v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
  v[8] = c.x, v[9] = c.y, v[10] = c.z, v[11] = c.w;
  v[12] = d.x, v[13] = d.y, v[14] = d.z, v[15] = d.w;
}
__device__ __forceinline__ uint32_t scale_mul2(uint32_t sc) {
  // fp16 pair holding 2^(sc-127): normal for sc in [113, 142], subnormal down to sc = 103, zero below
  const int f = (int)sc - 112;
  uint32_t h;
  if (f >= 1)
    h = (uint32_t)min(f, 30) << 10;
  else
    h = sc >= 103 ? (1u << (sc - 103)) : 0u;
  return h | (h << 16);
}


template <int MODE, int NT>
struct MoeSmem {
  static constexpr int kMats = 1;  // GEMM1 packs 64 gate rows and the 64 matching up rows into one 128-row tile
  static constexpr int kPackedBytes = kMats * kRowsTile * 128;  // per packed stage (256 K elements)
  static constexpr int kBBytes = 2 * NT * 128;                  // route rows of one 128-wide K chunk (two swizzle atoms)
  // A chunk (128 K elements, half a packed stage) is the unit handed from the builders to the MMA issuers.  Its
  // dequantised weights live in tensor memory ([128 lanes x 128 fp16] = 64 columns per matrix); only the packed
  // stages and the route rows use shared memory.  The packed ring keeps >= 64 KiB per SM in flight (HBM latency).
  static constexpr int kPStages = 8;
  static constexpr int kOBufs = 4;
  static constexpr int kXchBytes = MODE == 1 ? 2 * 64 * NT * 4 : 0;  // GEMM1 epilogue: up rows handed to the gate warps
  static constexpr int kTotal = kPStages * kPackedBytes + kOBufs * kBBytes + kXchBytes + 1024 + 512;
  static_assert(kTotal <= 227 * 1024, "shared memory budget");
  // Two accumulators per tile in both modes (gate/up, or the even/odd chunks of GEMM2), one per MMA issuer, and
  // two such pairs so that the epilogue of one tile overlaps the MMAs of the next.  NT = 64 is the widest tile for
  // which this and the operand buffers fit the 512 columns.
  static constexpr int kAccBufs = 2;
  static_assert(NT == 32 || NT == 64, "route tile");
  static constexpr int kAccCols = kAccBufs * 2 * NT;
  static constexpr int kACols = kMats * 64;
  static constexpr int kUsedCols = kAccCols + kOBufs * kACols;
  static constexpr uint32_t kTmemCols = kUsedCols <= 32 ? 32 : kUsedCols <= 64 ? 64 : kUsedCols <= 128 ? 128
                                        : kUsedCols <= 256 ? 256 : 512;
  static_assert(kUsedCols <= 512, "tensor memory budget");
};

// MODE 1: a work item is (route tile, 64 intermediate indices): TMEM lanes 0..63 hold the gate rows, lanes 64..127 the
//         up rows of the same indices, so GEMM1 has as many MMAs per byte as GEMM2 and twice as many (half-size) work
//         items to balance over the SMs.  act[pos, j] = fp16(bf16(silu(min(g,L)) * clamp(u,+-L))), w13 [E, 2I, K/2].
// MODE 2: D -> out[route, h] = bf16(bf16(acc) * bf16(w_route)), weights w2 [E, H, K/2].
//
// Why this shape.  A tcgen05.mma with M = 128, K = 16 costs about 64 cycles whatever N <= 128 is (it streams the
// 4 KiB A operand), so with a handful of routes per expert the tensor pipe, not HBM, bounds the kernel at 32 weight
// elements per cycle per SM, and everything else has to hide behind it:
//   * hand-offs happen in 128-element chunks, one tcgen05.commit per 8 MMAs of an issuer;
//   * two issuer threads feed the pipe (GEMM1: gate and up matrix; GEMM2: even and odd chunks into two accumulators
//     that the epilogue adds), so the per-chunk bookkeeping of one overlaps the MMAs of the other, and each polls the
//     barrier of its next chunk while its last MMAs of the current one are still queueing;
//   * every other waiting warp sleeps between polls (a polling warp takes issue slots from the issuers), and a warp
//     makes one mbarrier arrival, not 32.
template <int MODE, int NT>
__global__ void __launch_bounds__(kThreads, 1)
moe_gemm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                const uint8_t* __restrict__ scales, const PlanHeader* __restrict__ hdr, const int* __restrict__ tiles,
                const int* __restrict__ sorted_route, const float* __restrict__ sorted_w,
                __nv_bfloat16* __restrict__ out, int K, int rows_per_expert /*I (mode1) or H (mode2)*/,
                int ld_out, float limit) {
  using S = MoeSmem<MODE, NT>;
  constexpr int kOBufs = S::kOBufs, kPStages = S::kPStages, kAccBufs = S::kAccBufs;
  constexpr uint32_t kIdesc = umma_idesc(128, NT, 0, 0);  // fp16 x fp16 -> fp32
  constexpr int kSleep = 64;                              // ns between polls of the non-critical waits
  constexpr int kIssuerWarp1 = kThreads / 32 - 1, kRowProducerWarp = kThreads / 32 - 2;
  constexpr bool kDual = true;  // two MMA issuer threads
  extern __shared__ uint8_t moe_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(moe_smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* packed = smem;
  uint8_t* bbuf = smem + kPStages * S::kPackedBytes;
  float* xch = reinterpret_cast<float*>(bbuf + kOBufs * S::kBBytes);  // GEMM1 epilogue exchange (kXchBytes)
  uint64_t* bars = reinterpret_cast<uint64_t*>(bbuf + kOBufs * S::kBBytes + S::kXchBytes);
  uint64_t* pfull = bars;               // [kPStages]  packed stage landed
  uint64_t* pempty = pfull + kPStages;  // [kPStages]  packed stage read by every builder warp
  uint64_t* ofull = pempty + kPStages;  // [kOBufs]    chunk operands ready: weights in tensor memory + route rows landed
  uint64_t* oempty = ofull + kOBufs;    // [kOBufs]    the chunk's MMAs retired
  uint64_t* tfull = oempty + kOBufs;    // [2]         accumulators complete (one commit per issuer)
  uint64_t* tempty = tfull + 2;         // [2]         accumulators drained by the epilogue
  uint64_t* xfull = tempty + 2;         // [2]         GEMM1: the up warps' sums are in the exchange buffer
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(xfull + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row_tiles = rows_per_expert / (MODE == 1 ? 64 : kRowsTile);
  const int kstages = K / 256;
  const int nchunks = kstages * 2;
  const int scale_ld = K / 32;  // scale bytes per weight row

  if (threadIdx.x == 0) {
    for (int i = 0; i < kPStages; ++i) mbar_init(&pfull[i], 1), mbar_init(&pempty[i], kBuilders / 32);
    for (int i = 0; i < kOBufs; ++i)
      mbar_init(&ofull[i], kBuilders / 64 + 1), mbar_init(&oempty[i], 1);
    for (int i = 0; i < 2; ++i) mbar_init(&tfull[i], kDual ? 2 : 1), mbar_init(&tempty[i], 4), mbar_init(&xfull[i], 2);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, S::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();  // barriers and tensor memory are set up; from here on the kernel touches global memory
  pdl_launch_dependents();  // only after the own wait (common.cuh: programmatic dependent launch)
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t a_base = tmem_base + S::kAccCols;  // operand buffer b starts at column a_base + b * kACols
  const int total_work = hdr->num_tiles * row_tiles;

  if (warp == 0) {
    if (lane == 0) {  // packed weight stages
      int ps = 0;
      for (int wk = blockIdx.x; wk < total_work; wk += gridDim.x) {
        const int ct = wk / row_tiles, rt = wk % row_tiles;
        const int e = tiles[ct * 3];
        const int wrow = MODE == 1 ? e * 2 * rows_per_expert + rt * 64 : e * rows_per_expert + rt * kRowsTile;
        bool ok = true;
        for (int ks = 0; ks < kstages; ++ks, ++ps) {
          const int s = ps % kPStages;
          if (!mbar_wait<kSleep>(&pempty[s], ((ps / kPStages) & 1) ^ 1, abort_flag, 11)) { ok = false; break; }
          mbar_expect_tx(&pfull[s], S::kPackedBytes);
          uint8_t* dst = packed + s * S::kPackedBytes;
          tma_load_2d(dst, &tmW, &pfull[s], ks * 128, wrow);  // MODE 1: box of 64 rows (gate), MODE 2: 128 rows
          if (MODE == 1) tma_load_2d(dst + 64 * 128, &tmW, &pfull[s], ks * 128, wrow + rows_per_expert);  // up rows
        }
        if (!ok) break;
      }
    }
  } else if (warp == kRowProducerWarp) {
    if (lane == 0) {  // route rows (B operand) of one chunk: two 64-wide swizzle atoms
      int ob = 0;
      for (int wk = blockIdx.x; wk < total_work; wk += gridDim.x) {
        const int tok0 = tiles[(wk / row_tiles) * 3 + 1];
        bool ok = true;
        for (int ch = 0; ch < nchunks; ++ch, ++ob) {
          const int b = ob % kOBufs;
          if (!mbar_wait<kSleep>(&oempty[b], ((ob / kOBufs) & 1) ^ 1, abort_flag, 12)) { ok = false; break; }
          mbar_expect_tx(&ofull[b], S::kBBytes);
          tma_load_2d(bbuf + b * S::kBBytes, &tmX, &ofull[b], ch * 128, tok0);
          tma_load_2d(bbuf + b * S::kBBytes + NT * 128, &tmX, &ofull[b], ch * 128 + 64, tok0);
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1 || (kDual && warp == kIssuerWarp1)) {
    if (lane == 0) {
      // MMA issuer `iss`.  GEMM1: every chunk, matrix iss.  GEMM2: the chunks of parity iss, accumulator iss.
      const int iss = warp == 1 ? 0 : 1;
      const int step = kDual ? 2 : 1;
      int it = 0;
      long long ob0 = 0;  // global index of the work item's first chunk
      bool ok = true;
      for (int wk = blockIdx.x; wk < total_work && ok; wk += gridDim.x, ++it, ob0 += nchunks) {
        const int acc = it % kAccBufs;
        if (!mbar_wait(&tempty[acc], ((it / kAccBufs) & 1) ^ 1, abort_flag, 13)) break;
        const uint32_t d = tmem_base + acc * 2 * NT + iss * NT;
        const int ch0 = kDual ? iss : 0;
        bool ready = false;
        for (int ch = ch0; ch < nchunks; ch += step) {
          const long long ob = ob0 + ch;
          const int b = (int)(ob % kOBufs);
          if (!ready && !mbar_wait(&ofull[b], (uint32_t)(ob / kOBufs) & 1, abort_flag, 14)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a = a_base + b * S::kACols;
          const uint8_t* bt = bbuf + b * S::kBBytes;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            if (k == 6) {  // poll the next chunk's barrier while the last MMAs are still queueing
              const long long obn = ob + step;
              ready = ch + step < nchunks && mbar_try_wait(&ofull[obn % kOBufs], (uint32_t)(obn / kOBufs) & 1);
            }
            const uint64_t bd = umma_desc_k128(bt + (k >> 2) * (NT * 128), (k & 3) * 32);
            umma_f16_ta(d, a + k * 8, bd, kIdesc, (ch > ch0 || k > 0));
          }
          umma_commit(&oempty[b]);
        }
        if (ok) umma_commit(&tfull[acc]);
      }
    }
  } else if (warp < 6) {  // epilogue
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    int it = 0;
    for (int wk = blockIdx.x; wk < total_work; wk += gridDim.x, ++it) {
      const int acc = it % kAccBufs;
      const int ct = wk / row_tiles, rt = wk % row_tiles;
      const int tok0 = tiles[ct * 3 + 1], ntok = tiles[ct * 3 + 2];
      if (!mbar_wait<256>(&tfull[acc], (it / kAccBufs) & 1, abort_flag, 15)) break;
      tc_fence_after();
      const uint32_t d0 = lane_addr + acc * 2 * NT;
      // both accumulators (even / odd chunks) are added; then
      //   GEMM2: row = hidden index, scaled by the route weight;
      //   GEMM1: lanes 0..63 hold gate, lanes 64..127 up of the same 64 intermediate indices: the up warps hand their
      //          (bf16-rounded) sums over through shared memory, the gate warps apply SwiGLU and store.
      if (MODE == 2) {
        const int orow = rt * kRowsTile + r;
#pragma unroll 1
        for (int c0 = 0; c0 < NT; c0 += 16) {
          if (c0 >= ntok) break;
          uint32_t g[16], u[16];
          tmem_ld_32x16(d0 + c0, g);
          tmem_ld_32x16(d0 + NT + c0, u);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            if (c0 + c < ntok) {
              const int pos = tok0 + c0 + c;
              const __nv_bfloat16 y = f2bf(__uint_as_float(g[c]) + __uint_as_float(u[c]));
              const __nv_bfloat16 wv = f2bf(sorted_w[pos]);
              out[(size_t)sorted_route[pos] * ld_out + orow] = __hmul(y, wv);
            }
          }
        }
      } else {
        float* xq = xch + (size_t)acc * 64 * NT;  // [64 rows][NT], one buffer per accumulator pair
        const bool is_up = r >= 64;
        if (is_up) {
#pragma unroll 1
          for (int c0 = 0; c0 < NT; c0 += 16) {
            if (c0 >= ntok) break;
            uint32_t g[16], u[16];
            tmem_ld_32x16(d0 + c0, g);
            tmem_ld_32x16(d0 + NT + c0, u);
            tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 16; ++c)
              xq[(size_t)(r - 64) * NT + ((c0 + c + (r & 15)) & (NT - 1))] =
                  bf2f(f2bf(__uint_as_float(g[c]) + __uint_as_float(u[c])));
          }
        }
        if (is_up) {
          __syncwarp();
          if (lane == 0) mbar_arrive(&xfull[acc]);
        } else if (!mbar_wait(&xfull[acc], (it / kAccBufs) & 1, abort_flag, 19)) {
          break;
        }
        if (!is_up) {
          const int orow = rt * 64 + r;
#pragma unroll 1
          for (int c0 = 0; c0 < NT; c0 += 16) {
            if (c0 >= ntok) break;
            uint32_t g[16], u[16];
            tmem_ld_32x16(d0 + c0, g);
            tmem_ld_32x16(d0 + NT + c0, u);
            tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 16; ++c) {
              if (c0 + c < ntok) {
                float gv = bf2f(f2bf(__uint_as_float(g[c]) + __uint_as_float(u[c])));
                float uv = xq[(size_t)r * NT + ((c0 + c + (r & 15)) & (NT - 1))];
                if (limit > 0.f) {
                  gv = fminf(gv, limit);
                  uv = fminf(fmaxf(uv, -limit), limit);
                }
                const float a = gv / (1.f + expf(-gv)) * uv;
                // bf16 rounding of the activation, held as fp16 for the second GEMM's operand
                reinterpret_cast<__half*>(out)[(size_t)(tok0 + c0 + c) * ld_out + orow] =
                    __float2half_rn(bf2f(f2bf(a)));
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);  // one arrival per warp: arrivals on one barrier serialise
    }
  } else if (warp < 6 + kBuilders / 32) {
    // builders: two teams of 8 warps; team t dequantises the chunks of parity t (chunk t of every packed stage), so
    // one team builds while the other waits for its buffer.  A warp writes the tensor-memory lanes of its own
    // quarter (warp % 4), so a thread covers weight row (warp % 4) * 32 + lane and, by the warp's position in the
    // team, MODE 1: the chunk's 128 K elements of the gate (first four warps) or up matrix; MODE 2: the first or
    // second 64 K elements of the chunk.
    const int j = (warp - 6) & 7, team = (warp - 6) >> 3;
    const int quarter = warp & 3, half = j >> 2;
    const int r = quarter * 32 + lane;
    const uint32_t lane_addr = a_base + ((uint32_t)(quarter * 32) << 16);

    auto scale_row = [&](int wk) -> const uint8_t* {
      const int ct = wk / row_tiles, rt = wk % row_tiles;
      const size_t e = (size_t)tiles[ct * 3];
      const size_t wrow = MODE == 1 ? e * 2 * rows_per_expert + (r < 64 ? 0 : rows_per_expert) + rt * 64 + (r & 63)
                                    : e * rows_per_expert + rt * kRowsTile + r;
      return scales + wrow * scale_ld;
    };
    long long ps = 0;
    int wk = blockIdx.x;
    const uint8_t* srow = wk < total_work ? scale_row(wk) : nullptr;
    // the 4 scale bytes of this team's chunk are fetched one stage ahead: they come from HBM
    uint32_t scn = srow ? __ldg(reinterpret_cast<const uint32_t*>(srow + team * 4)) : 0u;
    for (; wk < total_work; wk += gridDim.x) {
      const int wk_next = wk + gridDim.x;
      const uint8_t* srow_next = wk_next < total_work ? scale_row(wk_next) : nullptr;
      bool ok = true;
      for (int ks = 0; ks < kstages; ++ks, ++ps) {
        const int s = (int)(ps % kPStages);
        const uint32_t sw = scn;
        if (ks + 1 < kstages)
          scn = __ldg(reinterpret_cast<const uint32_t*>(srow + (ks + 1) * 8 + team * 4));
        else if (srow_next)
          scn = __ldg(reinterpret_cast<const uint32_t*>(srow_next + team * 4));
        if (!mbar_wait<kSleep>(&pfull[s], (uint32_t)(ps / kPStages) & 1, abort_flag, 16)) { ok = false; break; }
        // chunk `team` of the stage = bytes [64 team, 64 team + 64) of the 128-byte packed row = 16-byte pieces
        // 4 team .. 4 team + 3 (swizzled by row), one scale byte each
        const uint8_t* prow = packed + s * S::kPackedBytes + r * 128;
        constexpr int kPieces = 2;
        const int piece0 = team * 4 + half * 2;
        uint4 p[kPieces];
#pragma unroll
        for (int i = 0; i < kPieces; ++i)
          p[i] = *reinterpret_cast<const uint4*>(prow + (((piece0 + i) ^ (r & 7)) << 4));
        const long long ob = ps * 2 + team;
        const int b = (int)(ob % kOBufs);
        if (!mbar_wait<kSleep>(&oempty[b], ((uint32_t)(ob / kOBufs) & 1) ^ 1, abort_flag, 17)) { ok = false; break; }
        tc_fence_after();
        const uint32_t dst = lane_addr + b * S::kACols + half * 32;
#pragma unroll
        for (int i = 0; i < kPieces; ++i) {
          const uint32_t sc = (sw >> (8 * (half * 2 + i))) & 0xff;
          uint32_t v[16];
          dequant8x4(p[i], scale_mul2(sc), v);
          tmem_st_32x16(dst + i * 16, v);
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&ofull[b]);
          // Release the packed stage only now, after its bytes were consumed by real instructions.  Releasing it
          // right after the loads were issued produced wrong sums: an arrival does not wait for loads whose results
          // nobody has used yet.
          mbar_arrive(&pempty[s]);
        }
      }
      if (!ok) break;
      srow = srow_next;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, S::kTmemCols);
}

// out[t] = bf16( float(bf16(sum_k local route rows)) + float(shared[t]) ); rows >= num_valid -> 0
// With xout != null the hyper-connection post mix is applied on the fly and xout [T,4,h] is written instead of out.
__global__ void moe_finalize_kernel(const __nv_bfloat16* __restrict__ yr, const int* __restrict__ route_pos,
                                    const __nv_bfloat16* __restrict__ shared, __nv_bfloat16* __restrict__ out,
                                    const int* __restrict__ num_valid, int topk, int h, const HcPostArgs hc) {
  pdl_entry();
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
    if (hc.res)
      hc_post_store8(o, hc, t, h, i);
    else
      *reinterpret_cast<uint4*>(out + (size_t)t * h + i) = o;
  }
}

// Fused combine: the per-token sum of the local routes (+ the shared expert) is this rank's partial of the layer
// output; it goes to the symmetric buffer and is reduced across ranks in the same kernel (protocol in comm.cuh).
// BIG: block-wise two-shot exchange for more than 256 tokens (prefill), see comm_big_two_shot.
template <bool BIG>
__global__ void __launch_bounds__(256) moe_finalize_ar_kernel(const __nv_bfloat16* __restrict__ yr,
                                                              const int* __restrict__ route_pos,
                                                              const __nv_bfloat16* __restrict__ shared,
                                                              __nv_bfloat16* __restrict__ out,
                                                              const int* __restrict__ num_valid, int topk, int h,
                                                              int t_rows, const HcPostArgs hc, const CommCtx comm) {
  pdl_entry();
  __shared__ int ok;
  const uint32_t epoch = comm_epoch(comm);
  const int parity = epoch & 1;
  __nv_bfloat16* mine = comm_data(comm, comm.rank, parity);
  const int nv = num_valid ? *num_valid : t_rows;
  // this rank's partial of rows [t0, t1): routes summed in fp32, rounded, + shared expert, into the parity buffer
  auto combine = [&](int t0, int t1) {
    for (int t = t0; t < t1; ++t) {
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
  };
  auto emit = [&](int t, int col, const uint4& v) {
    if (hc.res)
      hc_post_store8(v, hc, t, h, col);
    else
      *reinterpret_cast<uint4*>(out + (size_t)t * h + col) = v;
  };
  if constexpr (BIG) {
    comm_big_two_shot(comm, epoch, t_rows, h, &ok, combine, emit);
  } else {
    for (int t = blockIdx.x; t < t_rows; t += gridDim.x) combine(t, t + 1);
    __syncthreads();
    if (comm_use_multimem(comm, t_rows, h)) {
      const int t = blockIdx.x;
      if (t < t_rows) comm_row_multimem(comm, epoch, t, h, &ok, [&](int col, const uint4& v) { emit(t, col, v); });
    } else if (comm_use_two_shot(comm, t_rows, h)) {
      const int t = blockIdx.x;
      if (t < t_rows) comm_row_two_shot(comm, epoch, t, h, &ok, [&](int col, const uint4& v) { emit(t, col, v); });
    } else {
      if (threadIdx.x == 0) {
        comm_publish(comm, blockIdx.x, epoch);
        ok = comm_wait(comm, blockIdx.x, epoch) ? 1 : 0;
      }
      __syncthreads();
      if (ok) {
        for (int t = blockIdx.x; t < t_rows; t += gridDim.x) {
          for (int i = threadIdx.x * 8; i < h; i += blockDim.x * 16) {
            const int i1 = i + blockDim.x * 8;
            uint4 o0, o1;
            if (i1 < h) {
              comm_reduce16x2(comm, parity, (size_t)t * h + i, (size_t)t * h + i1, o0, o1);
              emit(t, i1, o1);
            } else {
              o0 = comm_reduce16(comm, parity, (size_t)t * h + i);
            }
            emit(t, i, o0);
          }
        }
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) comm_finish(comm, gridDim.x);
}

// Combine with a reduce-scatter instead of an all-reduce (row-sharded layer, comm.cuh): CTA t sums the local routes of
// token t (+ the shared expert) like moe_finalize_kernel and stores the partial row straight into the buffer of the
// rank that owns row t; the last row of a 128-row block raises the block's flag at the owner, whose
// sp_rs_reduce_kernel adds the ranks' partials (and applies the hyper-connection post mix).
__global__ void __launch_bounds__(256) moe_finalize_rs_kernel(const __nv_bfloat16* __restrict__ yr,
                                                              const int* __restrict__ route_pos,
                                                              const __nv_bfloat16* __restrict__ shared, int topk, int h,
                                                              int t_rows, const SpCtx sp, int* __restrict__ counters) {
  pdl_entry();
  const int t = blockIdx.x;
  const int rpr = sp.rows_per_rank, owner = t / rpr, blk = t >> 7;
  __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(sp.peer[owner] + sp.rs_off) +
                       ((size_t)sp.rank * rpr + (t - owner * rpr)) * h;
  for (int i = threadIdx.x * 8; i < h; i += blockDim.x * 8) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
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
    const __nv_bfloat162* spv = reinterpret_cast<const __nv_bfloat162*>(&su);
    uint4 o;
    __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 r2 = __bfloat1622float2(__floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]));
      const float2 s2 = __bfloat1622float2(spv[j]);
      po[j] = __floats2bfloat162_rn(r2.x + s2.x, r2.y + s2.y);
    }
    st_bulk16(dst + i, o);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const int rows_in_blk = min(128, t_rows - blk * 128);
    if (atomicAdd(&counters[blk], 1) == rows_in_blk - 1) {
      counters[blk] = 0;
      __threadfence_system();
      st_relaxed_sys(sp_flag(sp, owner, kSpRS, sp.rank, (blk * 128 - owner * rpr) >> 7), sp.seq);
    }
  }
}

template <int MODE, int NT>
int launch_moe_gemm(const void* w, const uint8_t* scales, const void* x, int x_rows, const PlanHeader* hdr,
                    const int* tiles, const int* sorted_route, const float* sorted_w, void* out, int e_local, int K,
                    int rows_per_expert, int ld_out, float limit, int num_sms, cudaStream_t st) {
  using S = MoeSmem<MODE, NT>;
  CUtensorMap tmW, tmX;
  const uint64_t wrows = (uint64_t)e_local * (MODE == 1 ? 2 : 1) * rows_per_expert;
  if (dsv4_make_tmap_2d(&tmW, w, 0, (uint64_t)K / 2, wrows, (uint64_t)K / 2, 128, MODE == 1 ? 64 : kRowsTile, 3))
    return 201;
  if (dsv4_make_tmap_2d(&tmX, x, 1, (uint64_t)K, (uint64_t)x_rows, (uint64_t)K * 2, 64, NT, 3)) return 202;
  auto kern = moe_gemm_kernel<MODE, NT>;
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal) != cudaSuccess) return 203;
    set = true;
  }
  dsv4_launch(kern, num_sms, kThreads, S::kTotal, st, tmW, tmX, scales, hdr, tiles, sorted_route, sorted_w, (__nv_bfloat16*)out,
                                            K, rows_per_expert, ld_out, limit);
  return (int)cudaGetLastError();
}

}  // namespace

DSV4_API int dsv4_moe_topk(const float* scores, const float* bias, const int* tid2eid, const int* token_ids,
                           const int* num_valid, int* idx, float* wts, int t, int e, int k, float scaling, int scoring,
                           int n_part, long long part_stride, cudaStream_t st) {
  if (t <= 0) return 0;
  if (e > 512 || k > 32 || n_part < 1) return 210;
  // one warp per token, two warps per CTA: a decode batch of 128 tokens then covers 64 SMs instead of 16
  dsv4_launch(moe_topk_kernel, (t * 32 + 63) / 64, 64, 0, st, scores, bias, tid2eid, token_ids, num_valid, idx, wts, t,
              e, k, scaling, scoring, n_part, part_stride);
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
  dsv4_launch(moe_plan_kernel, 1, 1024, smem, st, idx, wts, routes, e_local, base, nt, hdr, tiles, sorted_route, route_pos,
                                         sorted_w);
  return (int)cudaGetLastError();
}

DSV4_API int dsv4_moe_permute(const void* x, void* xs, const int* plan, int routes, int max_tiles, int topk, int h,
                              cudaStream_t st) {
  if (routes <= 0) return 0;
  const PlanHeader* hdr = reinterpret_cast<const PlanHeader*>(plan);
  const int* sorted_route = plan + 4 + 3 * max_tiles;
  dsv4_launch(moe_permute_kernel, routes, 128, 0, st, (const uint4*)x, (uint4*)xs, sorted_route, hdr, topk, h / 8);
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
  if (mode == 1 && nt == 64) MOE_LAUNCH(1, 64);
  if (mode == 2 && nt == 32) MOE_LAUNCH(2, 32);
  if (mode == 2 && nt == 64) MOE_LAUNCH(2, 64);
#undef MOE_LAUNCH
  return 221;
}

// res / post / comb / xout (all null, or all given): apply the hyper-connection post mix to the combined output and
// write the new residual streams xout [t, 4, h] instead of out.
DSV4_API int dsv4_moe_finalize(const void* yr, const int* plan, int routes, int max_tiles, const void* shared, void* out,
                               const int* num_valid, int t, int topk, int h, const void* res, const float* post,
                               const float* comb, void* xout, cudaStream_t st) {
  if (t <= 0) return 0;
  if (xout && (!res || !post || !comb)) return 231;
  const int* route_pos = plan + 4 + 3 * max_tiles + routes;
  dsv4_launch(moe_finalize_kernel, t, 256, 0, st, (const __nv_bfloat16*)yr, route_pos, (const __nv_bfloat16*)shared,
              (__nv_bfloat16*)out, num_valid, topk, h,
              HcPostArgs{xout ? (const __nv_bfloat16*)res : nullptr, post, comb, (__nv_bfloat16*)xout});
  return (int)cudaGetLastError();
}

// Combine + reduce-scatter (see moe_finalize_rs_kernel).  counters: >= ceil(t / 128) zero ints.  dsv4_sp_rs_reduce on
// every rank must follow.
DSV4_API int dsv4_moe_finalize_rs(const void* yr, const int* plan, int routes, int max_tiles, const void* shared, int t,
                                  int topk, int h, const SpCtx* sp, int* counters, cudaStream_t st) {
  if (t <= 0) return 0;
  if (h % 8 || h != sp->hidden || sp->rows_per_rank % 128 || !shared) return 232;
  const int* route_pos = plan + 4 + 3 * max_tiles + routes;
  dsv4_launch(moe_finalize_rs_kernel, t, 256, 0, st, (const __nv_bfloat16*)yr, route_pos, (const __nv_bfloat16*)shared,
              topk, h, t, *sp, counters);
  return (int)cudaGetLastError();
}

DSV4_API int dsv4_moe_finalize_allreduce(const void* yr, const int* plan, int routes, int max_tiles, const void* shared,
                                         void* out, const int* num_valid, int t, int topk, int h, const void* res,
                                         const float* post, const float* comb, void* xout, const CommCtx* comm,
                                         cudaStream_t st) {
  if (t <= 0) return 0;
  if (h % 8 || (long long)t * h * 2 > comm->data_bytes) return 230;
  if (xout && (!res || !post || !comb)) return 231;
  const int* route_pos = plan + 4 + 3 * max_tiles + routes;
  const HcPostArgs hc{xout ? (const __nv_bfloat16*)res : nullptr, post, comb, (__nv_bfloat16*)xout};
  if (comm_host_use_big(*comm, t))
    dsv4_launch(moe_finalize_ar_kernel<true>, comm_big_grid(t), 256, 0, st, (const __nv_bfloat16*)yr, route_pos,
                (const __nv_bfloat16*)shared, (__nv_bfloat16*)out, num_valid, topk, h, t, hc, *comm);
  else
    dsv4_launch(moe_finalize_ar_kernel<false>, t < 1024 ? t : 1024, 256, 0, st, (const __nv_bfloat16*)yr, route_pos,
                (const __nv_bfloat16*)shared, (__nv_bfloat16*)out, num_valid, topk, h, t, hc, *comm);
  return (int)cudaGetLastError();
}
