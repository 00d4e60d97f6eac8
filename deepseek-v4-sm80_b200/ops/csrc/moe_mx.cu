// Routed experts on the block-scaled tensor-core path: packed-FP4 weights with their e8m0 group scales go from HBM to
// the MMA untouched (tcgen05.mma kind::mxf8f6f4, block_scale), no dequantisation pass and K = 32 per instruction.
//
// Activations stay bf16-exact.  A bf16 value has 8 significant bits; it is written as hi + lo, two e4m3 values (4
// significant bits each) with one power-of-two scale per 32 K elements each: hi = e4m3(x / s_hi) rounded to nearest,
// lo = e4m3((x - hi s_hi) / s_lo) with s_lo = s_hi / 32.  The residual of the first rounding is a multiple of the
// bf16 value's last place and at most half a place of hi, so lo holds it exactly for every element within 2^14 of its
// block's largest magnitude (smaller ones keep an absolute error below 2^-22 of that magnitude, far under the fp32
// accumulation noise of the dot product).  hi and lo are two neighbouring columns of the MMA's N dimension (rows
// 2 r and 2 r + 1 of the B operand) that the epilogue adds:
//   D[row, n] = sum_k W[row, k] sw[row, k / 32] * X[n, k] sx[n, k / 32],   y[row, route] = D[row, 2 route] + D[row, 2 route + 1]
// This is the same product the reference's W4A16 path computes (python/minisgl/kernel/marlin_wna16.py:288-356:
// bf16 activations, exact FP4 dequantisation, fp32 accumulation), without the fp16 range limit of the f16-kind form.
//
// Weights are re-tiled once at load time: the 128 rows x 128 K elements that one pipeline stage consumes are 8 KiB of
// consecutive bytes ([expert][row tile][K chunk][128 rows][64 bytes]).  Read in place from the checkpoint layout, a
// stage would be 128 pieces of 64 bytes, 2 KiB (one weight row) apart, and all CTAs would walk the same byte offset
// of their rows at the same time: measured, that pattern stopped at 0.42 of the HBM copy rate with the DRAM channels
// unevenly loaded, whatever the kernel around it did.
//
// "swap-AB" as in moe.cu: the 128 weight rows of a work item sit on the TMEM lanes, routes are the N dimension.
// With a handful of routes per expert an instruction does little arithmetic, so what bounds the kernel is how fast
// instructions are issued, not the tensor pipe.  Measured on one CTA (M = 128, K = 32, this MMA kind): one thread
// issues an MMA every 68 cycles whatever N <= 128 is, two threads together every 39 (N = 16) to 64 cycles (N = 128,
// the pipe's own rate), a TMA or bulk copy costs its issuing thread about 70 cycles.  Inside this kernel, with one
// CTA per SM and 256-element stages, the issuer spent 785 cycles on a stage (8 MMAs, 4 scale copies) plus 165 on the
// barrier wait and the commit: more than the 735 cycles in which HBM delivers the stage's 17 KiB to one SM.
// Hence TWO CTAs PER SM, each with half the shared memory and one K chunk (128 elements, 8 KiB of packed weights) per
// stage: two independent issuers share the tensor pipe and together outrun HBM for narrow route tiles; for wide
// tiles (NT = 64, prefill: N = 128, where an MMA takes the pipe 64 cycles) they keep the pipe busy, and one CTA's
// epilogue runs under the other's MMAs (a wide tile has one accumulator set per CTA, a narrow one two).
// One thread issues all MMAs of a CTA.  (A second issuing thread in the same CTA, with its own accumulator and scale
// columns, stages alternating between the two, was tried twice, the second time with the accumulators on 32-column
// boundaries: right sums while the weights came from a warm L2, wrong sums and then a launch failure as soon as the
// issuers had to wait for HBM.  The cause was not found by reading, so a CTA has one issuer.)
// Warp roles per CTA (192 threads): warp 0 TMA producer (weights through a 4-bit "unpack" tensor map: 16 nibbles
// land in 16 bytes of shared memory, the operand form of this MMA kind), warp 1 tcgen05.cp of the scales into tensor
// memory + tcgen05.mma, warps 2-5 epilogue.
#include "common.cuh"

namespace {

constexpr int kMxThreads = 192;

struct MxPlanHeader {  // first 16 bytes of the plan buffer (moe.cu: PlanHeader)
  int num_tiles;
  int num_routes_local;
  int pad0, pad1;
};

// ue8m0 exponent bytes of a 32-element block whose largest magnitude is amax: hi values land in (-256, 256)
__device__ __forceinline__ void mx_block_exps(float amax, int& eh, int& el) {
  const int ef = (int)((__float_as_uint(amax) >> 23) & 0xff);
  eh = min(max(ef - 7, 5), 253);
  el = eh - 5;
}
__device__ __forceinline__ float e4m3_to_float(uint32_t b) {
  const __half_raw hr = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&hr));
}
// x (a bf16 value held in fp32) -> (hi, lo) bytes under the block exponents
__device__ __forceinline__ void mx_split(float x, int eh, int el, uint32_t& hi, uint32_t& lo) {
  const float inv_h = __uint_as_float((uint32_t)(254 - eh) << 23), s_h = __uint_as_float((uint32_t)eh << 23);
  const float inv_l = __uint_as_float((uint32_t)(254 - el) << 23);
  hi = __nv_cvt_float_to_fp8(x * inv_h, __NV_SATFINITE, __NV_E4M3);
  const float r = x - e4m3_to_float(hi) * s_h;
  lo = __nv_cvt_float_to_fp8(r * inv_l, __NV_SATFINITE, __NV_E4M3);
}
// byte offset of (row n, K block kb) inside a 512-byte scale block of 128 rows x 4 K blocks
__device__ __forceinline__ int sf_offset(int n, int kb) { return (n & 31) * 16 + (n >> 5) * 4 + kb; }

// xq[2 pos] = hi row, xq[2 pos + 1] = lo row of x[sorted_route[pos] / topk]; the block exponents go into the scale
// block of the position's route tile: sf[tile][K / 128][512] at rows 2 n and 2 n + 1, n = pos - tile start.
__global__ void __launch_bounds__(128) moe_mx_permute_kernel(const __nv_bfloat16* __restrict__ x,
                                                             uint8_t* __restrict__ xq, uint8_t* __restrict__ sf,
                                                             const MxPlanHeader* __restrict__ hdr,
                                                             const int* __restrict__ tiles,
                                                             const int* __restrict__ sorted_route, int topk, int h,
                                                             int routes, int max_tiles, int nt) {
  pdl_entry();
  const int pos = blockIdx.x;
  if (pos >= hdr->num_routes_local) return;
  if (hdr->num_tiles < 1 || hdr->num_tiles > max_tiles || hdr->num_routes_local > routes) {  // a plan from other sizes
    if (threadIdx.x == 0) dsv4_set_error(DSV4_ERR_BAD_INDEX, 31, hdr->num_tiles);
    return;
  }
  __shared__ int s_tile;
  if (threadIdx.x == 0) {  // the last tile that starts at or before pos (tiles are in position order)
    int lo = 0, hi = hdr->num_tiles - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (tiles[mid * 3 + 1] <= pos) lo = mid; else hi = mid - 1;
    }
    s_tile = lo;
  }
  __syncthreads();
  const int ti = s_tile, n = pos - tiles[ti * 3 + 1];
  const int tok = sorted_route[pos] / topk;
  if (n < 0 || n >= nt || sorted_route[pos] < 0 || sorted_route[pos] >= routes) {
    if (threadIdx.x == 0) dsv4_set_error(DSV4_ERR_BAD_INDEX, 32, pos);
    return;
  }
  const int nblk = h / 32, nchunks = h / 128;
  for (int blk = threadIdx.x; blk < nblk; blk += blockDim.x) {
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)tok * h + blk * 32);
    uint4 v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = src[i];
    const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(v);
    float f[32], amax = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) f[i] = bf2f(b[i]), amax = fmaxf(amax, fabsf(f[i]));
    int eh, el;
    mx_block_exps(amax, eh, el);
    uint32_t wh[8] = {0, 0, 0, 0, 0, 0, 0, 0}, wl[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      uint32_t hb, lb;
      mx_split(f[i], eh, el, hb, lb);
      wh[i >> 2] |= hb << (8 * (i & 3));
      wl[i >> 2] |= lb << (8 * (i & 3));
    }
    uint4* dh = reinterpret_cast<uint4*>(xq + (size_t)(2 * pos) * h + blk * 32);
    uint4* dl = reinterpret_cast<uint4*>(xq + (size_t)(2 * pos + 1) * h + blk * 32);
    dh[0] = make_uint4(wh[0], wh[1], wh[2], wh[3]), dh[1] = make_uint4(wh[4], wh[5], wh[6], wh[7]);
    dl[0] = make_uint4(wl[0], wl[1], wl[2], wl[3]), dl[1] = make_uint4(wl[4], wl[5], wl[6], wl[7]);
    uint8_t* sb = sf + ((size_t)ti * nchunks + (blk >> 2)) * 512;
    sb[sf_offset(2 * n, blk & 3)] = (uint8_t)eh;
    sb[sf_offset(2 * n + 1, blk & 3)] = (uint8_t)el;
  }
}

template <int MODE, int NT>
struct MxSmem {
  static constexpr int kCtasPerSm = 2;
  static constexpr int kChunks = 1;                        // 128-element K chunks per pipeline stage
  static constexpr int kABytes = kChunks * 128 * 128;      // per chunk: 128 weight rows x 128 K elements, one byte each
  static constexpr int kBBytes = kChunks * 2 * NT * 128;   // per chunk: rows (hi, lo) x routes, 128 K elements (e4m3)
  static constexpr int kSfBytes = kChunks * 512;           // per chunk: scales of 128 rows x 4 K blocks
  static constexpr int kStageBytes = kABytes + kBBytes + 2 * kSfBytes;
  // what the stage's copies report to the mbarrier: the unpacking weight copy counts the packed bytes it read
  static constexpr int kStageTxBytes = kABytes / 2 + kBBytes + 2 * kSfBytes;
  // 8 KiB of packed weights per stage: 2 CTAs x 5 or 4 stages keep >= 64 KiB per SM in flight (HBM latency)
  static constexpr int kStages = NT <= 8 ? 5 : NT <= 32 ? 4 : 3;
  static constexpr int kAccSets = NT <= 32 ? 2 : 1;  // accumulator sets of a CTA (two: its epilogue overlaps its next MMAs)
  static constexpr int kPass = NT < 32 ? NT : 32;                   // GEMM1 epilogue: routes per pass
  static constexpr int kXchBytes = MODE == 1 ? 128 * kPass * 2 : 0;  // its exchange buffer, bf16 [128 rows][kPass]
  static constexpr int kTotal = kStages * kStageBytes + kXchBytes + 1024 + 512;
  static_assert(kCtasPerSm * (kTotal + 1024) <= 228 * 1024, "shared memory budget (1 KiB per CTA is reserved)");
  static_assert(NT == 8 || NT == 16 || NT == 32 || NT == 64, "route tile");
  static constexpr int kAccStride = 2 * NT;  // columns of one accumulator set: [128 x (hi, lo) x NT]
  static constexpr int kAccCols = kAccSets * kAccStride;
  static constexpr int kSfCols = 2 * kChunks * 8;  // two buffers of kChunks x (SFA 4 + SFB 4) columns
  static constexpr int kUsedCols = kAccCols + kSfCols;
  static constexpr uint32_t kTmemCols = kUsedCols <= 64 ? 64 : kUsedCols <= 128 ? 128 : kUsedCols <= 256 ? 256 : 512;
  static_assert(kUsedCols <= 512, "tensor memory budget");
};

// MODE 1: work item = (route tile, 64 intermediate indices); lanes 0..63 hold the gate rows, lanes 64..127 the up rows
//         of the same indices.  The epilogue rounds both sums to bf16, applies the clamped SwiGLU, rounds to bf16 and
//         writes the result in the hi / lo form with its block exponents: the second GEMM's B operand.
//         w13 tiles [E, I/64, K/128, 128, 64 B] (rows 0..63 gate, 64..127 up), sfa [E, I/64, K/128, 512].
// MODE 2: D -> out[route, h] = bf16(bf16(acc) * bf16(w_route)); w2 tiles [E, H/128, K/128, 128, 64 B], sfa alike.
template <int MODE, int NT>
__global__ void __launch_bounds__(kMxThreads, 2)
moe_mx_gemm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                   const uint8_t* __restrict__ sfa, const uint8_t* __restrict__ sfb,
                   const MxPlanHeader* __restrict__ hdr, const int* __restrict__ tiles,
                   const int* __restrict__ sorted_route, const float* __restrict__ sorted_w, void* __restrict__ out,
                   uint8_t* __restrict__ sf_out, int K, int rows_per_expert /*I (mode 1) or H (mode 2)*/, int ld_out,
                   float limit, int e_local, int routes, int max_tiles) {
  using S = MxSmem<MODE, NT>;
  constexpr int kStages = S::kStages, kChunks = S::kChunks, kAccSets = S::kAccSets;
  constexpr uint32_t kIdesc = umma_idesc_mx(128, 2 * NT, 5, 0);  // e2m1 x e4m3, ue8m0 scales
  extern __shared__ uint8_t mx_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(mx_smem_raw) + 1023) & ~uintptr_t(1023));
  __nv_bfloat16* xch = reinterpret_cast<__nv_bfloat16*>(smem + kStages * S::kStageBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * S::kStageBytes + S::kXchBytes);
  uint64_t* full = bars;             // [kStages] stage landed
  uint64_t* empty = full + kStages;  // [kStages] the stage's MMAs and scale copies retired
  uint64_t* tfull = empty + kStages;  // [2] accumulator set complete (one commit per issuer)
  uint64_t* tempty = tfull + 2;       // [2] accumulator set drained by the four epilogue warps
  uint64_t* xfull = tempty + 2;       // [2] GEMM1 epilogue: [0] a pass' sums are in the exchange buffer, [1] they were read
  uint64_t* drain = xfull + 2;        // [1] only after a wait ran out: the MMAs in flight have retired
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(drain + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row_tiles = rows_per_expert / (MODE == 1 ? 64 : 128);
  const int nchunks = K / 128;
  const int nstages = nchunks / kChunks;  // stages per work item

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) mbar_init(&full[i], 1), mbar_init(&empty[i], 1);
    for (int i = 0; i < 2; ++i)
      mbar_init(&tfull[i], 1), mbar_init(&tempty[i], 4), mbar_init(&xfull[i], 4);
    mbar_init(drain, 1);
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
  pdl_wait();  // from here on the kernel touches global memory
  pdl_launch_dependents();  // only after the own wait (common.cuh: programmatic dependent launch)
  const uint32_t tmem_base = *tmem_holder;
  // every index below comes from the plan: a plan that does not fit these buffers is reported and skipped as a whole
  const bool plan_ok = hdr->num_tiles >= 0 && hdr->num_tiles <= max_tiles && hdr->num_routes_local <= routes;
  if (!plan_ok && threadIdx.x == 0) dsv4_set_error(DSV4_ERR_BAD_INDEX, 33, hdr->num_tiles);
  const int total_work = plan_ok ? hdr->num_tiles * row_tiles : 0;
  // one tile's fields: expert in range, its positions inside the route buffers
  auto tile_ok = [&](int ct) {
    const int e = tiles[ct * 3], t0 = tiles[ct * 3 + 1], n = tiles[ct * 3 + 2];
    return e >= 0 && e < e_local && t0 >= 0 && n >= 1 && n <= NT && t0 + n <= routes;
  };

  if (warp == 0) {
    if (lane == 0) {
      long long ps = 0;
      bool ok = true;
      for (int wk = blockIdx.x; wk < total_work && ok; wk += gridDim.x) {
        const int ct = wk / row_tiles, rt = wk % row_tiles;
        if (!tile_ok(ct)) {
          dsv4_set_error(DSV4_ERR_BAD_INDEX, 34, ct);
          *abort_flag = 1;
          break;
        }
        const int e = tiles[ct * 3], tok0 = tiles[ct * 3 + 1];
        const long long wrow = ((long long)e * row_tiles + rt) * nchunks * 128;  // first row of the item's first chunk
        const uint8_t* sa = sfa + ((size_t)e * row_tiles + rt) * nchunks * 512;
        const uint8_t* sb = sfb + (size_t)ct * nchunks * 512;
        for (int sg = 0; sg < nstages; ++sg, ++ps) {
          const int s = (int)(ps % kStages);
          if (!mbar_wait(&empty[s], ((uint32_t)(ps / kStages) & 1) ^ 1, abort_flag, 21)) { ok = false; break; }
          uint8_t* st = smem + s * S::kStageBytes;
          mbar_expect_tx(&full[s], S::kStageTxBytes);
          tma_load_2d(st, &tmW, &full[s], 0, (int)(wrow + sg * (kChunks * 128)));  // 16 KiB of consecutive bytes
#pragma unroll
          for (int c = 0; c < kChunks; ++c)
            tma_load_2d(st + S::kABytes + c * (2 * NT * 128), &tmX, &full[s], (sg * kChunks + c) * 128, 2 * tok0);
          bulk_load(st + S::kABytes + S::kBBytes, sa + (size_t)sg * S::kSfBytes, S::kSfBytes, &full[s]);
          bulk_load(st + S::kABytes + S::kBBytes + S::kSfBytes, sb + (size_t)sg * S::kSfBytes, S::kSfBytes, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      long long ps0 = 0;  // ring index of the work item's first stage
      int it = 0;
      bool ok = true;
      const uint32_t sf_base = tmem_base + S::kAccCols;
      for (int wk = blockIdx.x; wk < total_work && ok; wk += gridDim.x, ++it, ps0 += nstages) {
        const int acc = it % kAccSets;
        if (!mbar_wait(&tempty[acc], ((uint32_t)(it / kAccSets) & 1) ^ 1, abort_flag, 22)) break;
        tc_fence_after();
        const uint32_t d = tmem_base + acc * S::kAccStride;
        bool first = true;
        for (int sg = 0; sg < nstages; ++sg) {
          const long long ps = ps0 + sg;
          const int s = (int)(ps % kStages);
          if (!mbar_wait(&full[s], (uint32_t)(ps / kStages) & 1, abort_flag, 23)) { ok = false; break; }
          tc_fence_after();
          const uint8_t* st = smem + s * S::kStageBytes;
          const uint32_t sft = sf_base + (uint32_t)(ps & 1) * (kChunks * 8);  // the scale columns alternate per stage
          const uint64_t a0 = umma_desc_k128(st, 0), b0 = umma_desc_k128(st + S::kABytes, 0);
#pragma unroll
          for (int c = 0; c < kChunks; ++c) {
            tmem_cp_sf(sft + c * 8, st + S::kABytes + S::kBBytes + c * 512);
            tmem_cp_sf(sft + c * 8 + 4, st + S::kABytes + S::kBBytes + S::kSfBytes + c * 512);
          }
#pragma unroll
          for (int c = 0; c < kChunks; ++c) {
#pragma unroll
            for (int k = 0; k < 4; ++k)  // descriptors advance in 16-byte units: 32 bytes per K step
              umma_mx(d, a0 + (uint64_t)(c * (128 * 128 / 16) + k * 2), b0 + (uint64_t)(c * (2 * NT * 128 / 16) + k * 2),
                      kIdesc, k, sft + c * 8, sft + c * 8 + 4, !(first && c == 0 && k == 0));
          }
          first = false;
          umma_commit(&empty[s]);
        }
        if (ok) umma_commit(&tfull[acc]);
      }
    }
  } else if (warp < 6) {  // epilogue: warp w reads the TMEM lanes of quarter w % 4
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    int it = 0;
    [[maybe_unused]] int xph = 0;  // GEMM1: passes through the exchange buffer so far
    // hi + lo of 8 routes: 16 accumulator columns
    auto load8 = [&](uint32_t d0, int r0, float (&y)[8]) {
      uint32_t a[16];
      tmem_ld_32x16(d0 + 2 * r0, a);
      tmem_ld_wait();
#pragma unroll
      for (int c = 0; c < 8; ++c) y[c] = __uint_as_float(a[2 * c]) + __uint_as_float(a[2 * c + 1]);
    };
    for (int wk = blockIdx.x; wk < total_work; wk += gridDim.x, ++it) {
      const int acc = it % kAccSets;
      const int ct = wk / row_tiles, rt = wk % row_tiles;
      if (!tile_ok(ct)) break;  // the producer reports it and stops the CTA
      const int tok0 = tiles[ct * 3 + 1], ntok = tiles[ct * 3 + 2];
      if (!mbar_wait<256>(&tfull[acc], (uint32_t)(it / kAccSets) & 1, abort_flag, 24)) break;
      tc_fence_after();
      const uint32_t d0 = lane_addr + acc * S::kAccStride;
      if (MODE == 2) {
        const int orow = rt * 128 + r;
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out);
#pragma unroll 1
        for (int r0 = 0; r0 < NT; r0 += 8) {
          if (r0 >= ntok) break;
          float y[8];
          load8(d0, r0, y);
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            if (r0 + c < ntok) {
              const int pos = tok0 + r0 + c;
              const int route = sorted_route[pos];
              if (route >= 0 && route < routes)
                o[(size_t)route * ld_out + orow] = __hmul(f2bf(y[c]), f2bf(sorted_w[pos]));
              else
                dsv4_set_error(DSV4_ERR_BAD_INDEX, 35, pos);
            }
          }
        }
      } else {
        // SwiGLU and the hi / lo split, kPass routes at a time.  Step 1, all four warps: the bf16-rounded sums of
        // the pass go to shared memory, xs[row][route] (gate rows 0..63, up rows 64..127; a row's entries are rotated
        // by the row number, which spreads the lanes' column-wise stores over the banks).  Step 2, warps 0 and 1 of the
        // group: thread (block b, route) reads its 32 gate and 32 up values, applies the clamped SwiGLU, takes the
        // block's largest magnitude in registers and stores 32 hi and 32 lo bytes as two 16-byte pieces each.
        constexpr int kPass = S::kPass;
        bool dead = false;
#pragma unroll 1
        for (int p0 = 0; p0 < NT && !dead; p0 += kPass) {
          if (p0 >= ntok) break;
          // the readers of the pass before (of this or the previous work item) are done with xs
          if (xph > 0 && !mbar_wait(&xfull[1], (uint32_t)(xph - 1) & 1, abort_flag, 26)) { dead = true; break; }
#pragma unroll 1
          for (int r0 = p0; r0 < p0 + kPass; r0 += 8) {
            if (r0 >= ntok) break;
            float y[8];
            load8(d0, r0, y);
#pragma unroll
            for (int c = 0; c < 8; ++c) xch[r * kPass + ((r0 - p0 + c + r) & (kPass - 1))] = f2bf(y[c]);
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&xfull[0]);
          if (!mbar_wait(&xfull[0], (uint32_t)xph & 1, abort_flag, 25)) { dead = true; break; }
          const int n = p0 + lane;  // route of the tile
          if (q < 2 && lane < kPass && n < ntok) {
            const int b = q;
            float a[32], amax = 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int rg = b * 32 + i, ru = 64 + rg;
              float gv = bf2f(xch[rg * kPass + ((lane + rg) & (kPass - 1))]);
              float uv = bf2f(xch[ru * kPass + ((lane + ru) & (kPass - 1))]);
              if (limit > 0.f) {
                gv = fminf(gv, limit);
                uv = fminf(fmaxf(uv, -limit), limit);
              }
              a[i] = bf2f(f2bf(gv / (1.f + expf(-gv)) * uv));
              amax = fmaxf(amax, fabsf(a[i]));
            }
            int eh, el;
            mx_block_exps(amax, eh, el);
            uint32_t wh[8] = {0, 0, 0, 0, 0, 0, 0, 0}, wl[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              uint32_t hb, lb;
              mx_split(a[i], eh, el, hb, lb);
              wh[i >> 2] |= hb << (8 * (i & 3));
              wl[i >> 2] |= lb << (8 * (i & 3));
            }
            const int col0 = rt * 64 + b * 32;  // first intermediate index of the block
            uint8_t* act = reinterpret_cast<uint8_t*>(out);
            uint4* dh = reinterpret_cast<uint4*>(act + (size_t)(2 * (tok0 + n)) * ld_out + col0);
            uint4* dl = reinterpret_cast<uint4*>(act + (size_t)(2 * (tok0 + n) + 1) * ld_out + col0);
            dh[0] = make_uint4(wh[0], wh[1], wh[2], wh[3]), dh[1] = make_uint4(wh[4], wh[5], wh[6], wh[7]);
            dl[0] = make_uint4(wl[0], wl[1], wl[2], wl[3]), dl[1] = make_uint4(wl[4], wl[5], wl[6], wl[7]);
            uint8_t* sblk = sf_out + ((size_t)ct * (rows_per_expert / 128) + col0 / 128) * 512;
            const int kb = (col0 >> 5) & 3;
            sblk[sf_offset(2 * n, kb)] = (uint8_t)eh;
            sblk[sf_offset(2 * n + 1, kb)] = (uint8_t)el;
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&xfull[1]);
          ++xph;
        }
        if (dead) break;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // a wait ran out (the status word says where): before the tensor memory is freed and the CTA leaves, let the
    // MMAs already issued retire and the copies in flight land, each with a limit of its own
    if (warp == 1 && lane == 0) {
      umma_commit(drain);
      for (int i = 0; i < 20000 && !mbar_try_wait(drain, 0); ++i) __nanosleep(100);
    }
    if (threadIdx.x == 0)
      for (int i = 0; i < 100; ++i) __nanosleep(1000);
    tc_fence_before();
    __syncthreads();
  }
  if (warp == 1) tmem_dealloc(tmem_base, S::kTmemCols);
}

template <int MODE, int NT>
int launch_mx_gemm(const void* w, const uint8_t* sfa, const void* xq, const uint8_t* sfb, int x_rows,
                   const MxPlanHeader* hdr, const int* tiles, const int* sorted_route, const float* sorted_w, void* out,
                   uint8_t* sf_out, int e_local, int K, int rows_per_expert, int ld_out, float limit, int num_sms,
                   int max_tiles, cudaStream_t st) {
  using S = MxSmem<MODE, NT>;
  CUtensorMap tmW, tmX;
  // tile-major weights: every 128 rows x 64 bytes are one K chunk of one work item, chunks of an item follow each other
  const uint64_t wrows = (uint64_t)e_local * (rows_per_expert / (MODE == 1 ? 64 : 128)) * (K / 128) * 128;
  if (dsv4_make_tmap_2d(&tmW, w, 3, 128, wrows, 64, 128, S::kChunks * 128, 3)) return 241;
  if (dsv4_make_tmap_2d(&tmX, xq, 0, (uint64_t)K, (uint64_t)2 * x_rows, (uint64_t)K, 128, 2 * NT, 3)) return 242;
  auto kern = moe_mx_gemm_kernel<MODE, NT>;
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal) != cudaSuccess) return 243;
    // two CTAs per SM need the SM's whole shared-memory carveout
    cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
    set = true;
  }
  dsv4_launch(kern, num_sms * S::kCtasPerSm, kMxThreads, S::kTotal, st, tmW, tmX, sfa, sfb, hdr, tiles, sorted_route, sorted_w, out,
              sf_out, K, rows_per_expert, ld_out, limit, e_local, x_rows, max_tiles);
  return (int)cudaGetLastError();
}

}  // namespace

// x bf16 [t, h] -> xq uint8 [2 * routes, h] (rows 2 pos and 2 pos + 1: hi and lo of the route at position pos in
// expert order) and the per-tile scale blocks sf [max_tiles, h / 128, 512].  plan: the buffer dsv4_moe_plan filled.
DSV4_API int dsv4_moe_mx_permute(const void* x, void* xq, void* sf, const int* plan, int routes, int max_tiles, int topk,
                                 int h, int nt, cudaStream_t st) {
  if (routes <= 0) return 0;
  if (h % 128 || (nt != 8 && nt != 16 && nt != 32 && nt != 64)) return 240;
  const MxPlanHeader* hdr = reinterpret_cast<const MxPlanHeader*>(plan);
  const int* tiles = plan + 4;
  const int* sorted_route = tiles + 3 * max_tiles;
  dsv4_launch(moe_mx_permute_kernel, routes, 128, 0, st, (const __nv_bfloat16*)x, (uint8_t*)xq, (uint8_t*)sf, hdr, tiles,
              sorted_route, topk, h, routes, max_tiles, nt);
  return (int)cudaGetLastError();
}

// mode 1: xq / sfb = permuted tokens (K = H) -> out = act uint8 [2 * routes, I] (hi / lo rows), sf_out = its scale
//         blocks [max_tiles, I / 128, 512];  mode 2: xq / sfb = act (K = I) -> out = route rows bf16 [routes, H].
// w: packed FP4 in tiles [E, row tiles, K / 128, 128, 64 bytes] (32-byte aligned); sfa: the weight scales in 512-byte
// blocks [E, row tiles, K / 128, 512] (see the kernel).  nt: the route tile the plan was made with.
DSV4_API int dsv4_moe_mx_gemm(int mode, int nt, const void* w, const void* sfa, const void* xq, const void* sfb,
                              const int* plan, int routes, int max_tiles, void* out, void* sf_out, int e_local, int K,
                              int rows_per_expert, int ld_out, float limit, int num_sms, cudaStream_t st) {
  if (routes <= 0) return 0;
  if (K % 256 || rows_per_expert % 128 || (reinterpret_cast<uintptr_t>(w) & 31)) return 244;  // K: whole stages
  const MxPlanHeader* hdr = reinterpret_cast<const MxPlanHeader*>(plan);
  const int* tiles = plan + 4;
  const int* sorted_route = tiles + 3 * max_tiles;
  const float* sorted_w = reinterpret_cast<const float*>(sorted_route + 2 * routes);
#define MX_LAUNCH(M, N)                                                                                              \
  return launch_mx_gemm<M, N>(w, (const uint8_t*)sfa, xq, (const uint8_t*)sfb, routes, hdr, tiles, sorted_route,      \
                              sorted_w, out, (uint8_t*)sf_out, e_local, K, rows_per_expert, ld_out, limit, num_sms,   \
                              max_tiles, st)
  if (mode == 1 && nt == 8) MX_LAUNCH(1, 8);
  if (mode == 1 && nt == 16) MX_LAUNCH(1, 16);
  if (mode == 1 && nt == 32) MX_LAUNCH(1, 32);
  if (mode == 1 && nt == 64) MX_LAUNCH(1, 64);
  if (mode == 2 && nt == 8) MX_LAUNCH(2, 8);
  if (mode == 2 && nt == 16) MX_LAUNCH(2, 16);
  if (mode == 2 && nt == 32) MX_LAUNCH(2, 32);
  if (mode == 2 && nt == 64) MX_LAUNCH(2, 64);
#undef MX_LAUNCH
  return 245;
}
