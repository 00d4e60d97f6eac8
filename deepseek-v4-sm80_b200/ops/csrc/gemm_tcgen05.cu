// Dense projection GEMM for sm_100a:  out[M,N] = X[M,K] * W[N,K]^T  (both operands K-major).
//
// One CTA computes a 128 x BN output tile (or, with split-K, its share of the K range).  Warp 0 streams A/B k-tiles
// with TMA (128-byte swizzle) through a multi-stage mbarrier ring, warp 1 issues tcgen05.mma with the accumulator in
// tensor memory, warps 2-5 read the accumulator back with tcgen05.ld and write the result.
//
// Two operand formats:
//   * bf16 x bf16 (kind::f16), fp32 accumulate over the CTA's K range in one TMEM buffer.
//   * e4m3 x e4m3 with power-of-two block scales: activations carry one fp32 scale per (row, 128-wide K block),
//     weights one per (128 x 128) block.  The scales go to the tensor core as they are: the block-scaled MMA
//     (kind::mxf8f6f4.block_scale) multiplies every 32-element K group by 2^(ea + eb) from ue8m0 bytes in tensor memory
//     and accumulates the whole K range in ONE fp32 accumulator, i.e.  out = sum_kb sa[row,kb] * sw[nb,kb] * partial_kb
//     -- the arithmetic of the reference's "fake-quant activations x dequantised weights" path
//     (python/minisgl/models/deepseek_v4.py:145-149, :483) up to summation order -- without reading a partial product
//     back per K block (an earlier version promoted every 128-wide block through the epilogue warps, which bounded
//     the kernel at 0.33 us per k-tile and kept tiles at 32 columns: 0.16-0.2 of the HBM rate at 128 rows).  Before
//     the main loop the four epilogue warps turn this CTA's scales into 512-byte blocks in shared memory, one per
//     k-tile, holding byte(sa[row,kb]) + byte(sw[nb,kb]) - 127 for the tile's 128 rows (the weight scale is uniform
//     over a tile's columns, so it is folded into the row scale and the column-side scale is the constant 1).
//     Scales must be exact powers of two (they are: e8m0 weights, power-of-two activation quantisation); a scale with
//     mantissa bits is reported in the status word.
//
// Three launch extensions, all through blockIdx.z = batch * splits + split:
//   * batched: batch b reads A columns [b*a_col_pb, +K), B rows [b*b_row_pb, +N) and writes output columns
//     [b*out_col_pb, +N) -- the grouped low-rank output projection (wo_a) in one launch;
//   * split-K for skinny problems: every split writes its fp32 partial tile to a workspace, the last split to arrive
//     (per-tile counter) sums the partials in split order, so the result does not depend on arrival order;
//   * fused all-reduce: the epilogue publishes the partial tile to the rank's symmetric buffer and reduces the peers'
//     tiles over NVLink (comm.cuh).
#include "comm.cuh"

namespace {

constexpr int kBM = 128;
constexpr int kRowBytes = 128;  // one swizzle span per tile row

constexpr int kMaxKt = 64;  // fp8: k-tiles (128 elements each) of one CTA's K range whose scale blocks fit shared memory

template <int BN, bool FP8 = false>
struct GemmCfg {
  static constexpr int kStages = (BN >= 128) ? 5 : 6;
  static constexpr int kABytes = kBM * kRowBytes;
  static constexpr int kBBytes = BN * kRowBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // fp8: one 512-byte scale block per k-tile + the constant block of ones
  static constexpr int kSfBytes = FP8 ? (kMaxKt + 1) * 512 : 0;
  static constexpr int kSmemBytes = kStages * kStageBytes + kSfBytes + 1024 /*align*/ + 256 /*barriers*/;
};

struct GemmArgs {
  int M, N, K, ldo;
  const float* sa;     // [M, K/128] (fp8)
  const float* sb;     // [rows/128, K/128] (fp8), indexed with the batch's row offset
  int sb_ld;           // scale blocks per weight row block (= K/128 of the full weight)
  int accumulate_out;
  int a_col_pb, b_row_pb, out_col_pb;
  int splits;
  float* ws;           // [tiles][splits][128][BN] fp32 partials
  int* counters;       // [tiles], zero between launches
  int deposit_only;    // with a communicator: only write this rank's partial into the channel's symmetric buffer;
                       //   a following dsv4_allreduce(x = null) on the same channel reduces it
  int prefetch_b;      // the weight operand is not written by the kernel before this one: load it before pdl_wait()
  int cluster;         // > 0: the `splits` CTAs of a tile form one thread-block cluster and reduce over distributed
                       //      shared memory (no workspace, no atomics)
  long long partial_stride;  // > 0: split s writes its own partial product to out + s * partial_stride (no reduction;
                             //      the consumer kernel sums the splits in order)
  // Row-sharded exchange (comm.cuh, "row-sharded"): sp_mode 1 = the A operand is the gathered buffer: the TMA
  // producer waits for the flag of its 128-row block (raised by the block's owner) before loading A tiles;
  // sp_mode 2 = reduce-scatter epilogue: every partial row goes to its owner's buffer over NVLink and the last
  // column tile of a row block raises the block's flag at the owner.
  int sp_mode;
  int* sp_counters;          // [row blocks], zero between launches (sp_mode 2)
  SpCtx sp;
};

__device__ __forceinline__ void store_row_chunk(__nv_bfloat16* dst, const float* v, int ncols_valid) {
  if (ncols_valid >= 32 && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 p0 = __floats2bfloat162_rn(v[8 * i + 0], v[8 * i + 1]);
      __nv_bfloat162 p1 = __floats2bfloat162_rn(v[8 * i + 2], v[8 * i + 3]);
      __nv_bfloat162 p2 = __floats2bfloat162_rn(v[8 * i + 4], v[8 * i + 5]);
      __nv_bfloat162 p3 = __floats2bfloat162_rn(v[8 * i + 6], v[8 * i + 7]);
      uint4 u;
      u.x = *reinterpret_cast<uint32_t*>(&p0);
      u.y = *reinterpret_cast<uint32_t*>(&p1);
      u.z = *reinterpret_cast<uint32_t*>(&p2);
      u.w = *reinterpret_cast<uint32_t*>(&p3);
      reinterpret_cast<uint4*>(dst)[i] = u;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < ncols_valid) dst[i] = f2bf(v[i]);
  }
}
__device__ __forceinline__ void store_row_chunk(float* dst, const float* v, int ncols_valid) {
  if (ncols_valid >= 32 && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < ncols_valid) dst[i] = v[i];
  }
}

template <int BN, bool FP8, typename OutT>
__global__ void __launch_bounds__(192, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, OutT* __restrict__ out,
               const GemmArgs g, const CommCtx comm) {
  using Cfg = GemmCfg<BN, FP8>;
  constexpr int S = Cfg::kStages;
  constexpr int BK = FP8 ? 128 : 64;  // elements per k-tile (= 128 bytes)
  // one accumulator [128 x BN]; fp8 adds the scale columns: 4 for the constant column-side block, 2 x 4 for the row
  // scales of the k-tile in flight and the next one
  constexpr uint32_t kTmemCols = FP8 ? (BN <= 32 ? 64 : BN <= 64 ? 128 : 256) : (BN < 32 ? 32 : BN);
  constexpr uint32_t kIdesc = FP8 ? umma_idesc_mx(kBM, BN, 0, 0) : umma_idesc(kBM, BN, 1, 1);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint8_t* sf_all = smem + S * Cfg::kStageBytes;  // fp8: [nkt] row-scale blocks, then the block of ones
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + S * Cfg::kStageBytes + Cfg::kSfBytes);
  uint64_t* empty = full + S;
  uint64_t* tfull = empty + S;   // [8]
  uint64_t* tempty = tfull + 8;  // [8]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tempty + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  volatile int* sh_flag = reinterpret_cast<volatile int*>(tmem_holder + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int M = g.M, N = g.N;
  const int batch = blockIdx.z / g.splits, split = blockIdx.z % g.splits;
  const int n0 = blockIdx.x * BN;
  const int m0 = blockIdx.y * kBM;
  const int k_tiles = (g.K + BK - 1) / BK;
  const int kt_per = (k_tiles + g.splits - 1) / g.splits;
  const int kt0 = split * kt_per;
  const int nkt = max(min(kt0 + kt_per, k_tiles) - kt0, 0);

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 8; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 128);  // [0]: fp8, the 128 epilogue threads have written the scale blocks
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  // Barriers and tensor memory are set up.  The weight operand does not depend on the kernel before this one, so the
  // producer asks for the first ring of weight tiles BEFORE waiting for that kernel (under programmatic dependent
  // launch this CTA is already resident while it drains): their HBM latency is paid in the shadow of the previous
  // kernel.  Everything else (activation loads, scale reads, output writes) comes after pdl_wait().
  const int pre = g.prefetch_b ? (nkt < S ? nkt : S) : 0;
  if (warp == 0 && lane == 0) {
    const int by = batch * g.b_row_pb + n0;
    for (int i = 0; i < pre; ++i) {
      mbar_expect_tx(&full[i], Cfg::kStageBytes);
      tma_load_2d(tiles + i * Cfg::kStageBytes + Cfg::kABytes, &tmB, &full[i], (kt0 + i) * BK, by);
    }
  }
  pdl_wait();
  pdl_launch_dependents();  // only after the own wait (common.cuh: programmatic dependent launch)

  if (warp == 0) {
    if (lane == 0) {
      const int ax = batch * g.a_col_pb, by = batch * g.b_row_pb + n0;
      bool gate_ok = true;
      if (g.sp_mode == 1) {
        // all-gather fused into the load: the rows of this tile were pushed into the local gathered buffer by their
        // owner; wait for the owner's flag, then make its (generic-proxy) writes visible to the TMA reads
        const int owner = m0 / g.sp.rows_per_rank;
        if (owner != g.sp.rank)
          gate_ok = sp_wait_flag(sp_flag(g.sp, g.sp.rank, kSpAG, owner, m0 >> 7), g.sp.seq, owner, m0 >> 7);
        asm volatile("fence.proxy.async.global;" ::: "memory");
        if (!gate_ok) *abort_flag = 1;
      }
      for (int i = 0; i < nkt && gate_ok; ++i) {
        const int s = i % S;
        const uint32_t ph = (i / S) & 1;
        uint8_t* a = tiles + s * Cfg::kStageBytes;
        if (i < pre) {  // weights already requested above
          tma_load_2d(a, &tmA, &full[s], ax + (kt0 + i) * BK, m0);
          continue;
        }
        if (!mbar_wait<32>(&empty[s], ph ^ 1, abort_flag, 1)) break;
        mbar_expect_tx(&full[s], Cfg::kStageBytes);
        tma_load_2d(a, &tmA, &full[s], ax + (kt0 + i) * BK, m0);
        tma_load_2d(a + Cfg::kABytes, &tmB, &full[s], (kt0 + i) * BK, by);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t d = tmem_base;
      const uint32_t sfb_t = tmem_base + BN, sfa_t = tmem_base + BN + 4;  // scale columns behind the accumulator
      bool ok = true;
      if (FP8 && nkt > 0) {
        // the scale blocks of this CTA's K range are in shared memory once the epilogue warps have arrived
        ok = mbar_wait(&tempty[0], 0, abort_flag, 2);
        tc_fence_after();
        if (ok) tmem_cp_sf(sfb_t, sf_all + (size_t)nkt * 512);
      }
      for (int i = 0; i < nkt && ok; ++i) {
        const int s = i % S;
        const uint32_t ph = (i / S) & 1;
        if (!mbar_wait(&full[s], ph, abort_flag, 3)) break;
        tc_fence_after();
        const uint8_t* a = tiles + s * Cfg::kStageBytes;
        const uint8_t* bt = a + Cfg::kABytes;
        const uint32_t sfa_i = sfa_t + (uint32_t)(i & 1) * 4;
        if (FP8) tmem_cp_sf(sfa_i, sf_all + (size_t)i * 512);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint64_t ad = umma_desc_k128(a, k * 32);
          const uint64_t bd = umma_desc_k128(bt, k * 32);
          const uint32_t acc = (i > 0 || k > 0);
          if (FP8)
            umma_mx(d, ad, bd, kIdesc, k, sfa_i, sfb_t, acc);
          else
            umma_f16(d, ad, bd, kIdesc, acc);
        }
        umma_commit(&empty[s]);
      }
      if (nkt > 0) umma_commit(&tfull[0]);
    }
  } else {
    // epilogue warps 2..5 ; TMEM lane quarter = warp % 4
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int grow = m0 + row;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    const bool fused = comm.world > 1;
    uint32_t epoch = 0;
    OutT* part = out + (size_t)batch * g.out_col_pb + (g.partial_stride > 0 ? (size_t)split * g.partial_stride : 0);
    int ld_part = g.ldo;
    if (fused) {
      epoch = comm_epoch(comm);
      part = reinterpret_cast<OutT*>(comm_data(comm, comm.rank, epoch & 1));
      ld_part = N;
    }
    float acc[BN];
#pragma unroll
    for (int j = 0; j < BN; ++j) acc[j] = 0.f;
    bool ok = true;
    if (FP8 && g.sp_mode == 1) {
      // the activation scales are part of the gathered buffer: like the TMA producer, wait for the owner's flag of this
      // row block before reading them (one thread polls, the group's barrier hands the result to the others)
      if (warp == 2 && lane == 0) {
        const int owner = m0 / g.sp.rows_per_rank;
        bool gate_ok = true;
        if (owner != g.sp.rank)
          gate_ok = sp_wait_flag(sp_flag(g.sp, g.sp.rank, kSpAG, owner, m0 >> 7), g.sp.seq, owner, m0 >> 7);
        __threadfence();
        *sh_flag = gate_ok ? 1 : 0;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      __threadfence();
      ok = *sh_flag != 0;
      asm volatile("bar.sync 1, 128;" ::: "memory");  // sh_flag is reused by the split-K reduction below
    }
    if (FP8 && nkt > 0) {
      // scale blocks: block i, word (row % 32) * 4 + row / 32 = the byte ea(row, k-tile i) + eb(k-tile i) - 127 four
      // times (one per 32-element group of the tile); the block behind them is all 127 (2^0)
      const size_t sb_row = (size_t)((batch * g.b_row_pb + n0) >> 7) * g.sb_ld;
      const float* sa_row = g.sa + (size_t)(grow < M ? grow : 0) * k_tiles + kt0;
      uint32_t* blk = reinterpret_cast<uint32_t*>(sf_all) + (row & 31) * 4 + (row >> 5);
      bool pow2 = true;
      // sixteen k-tiles at a time: all their scale loads are in flight together (a dependent loop would pay the
      // global-memory latency once per k-tile, before the first MMA can be issued)
#pragma unroll 1
      for (int i0 = 0; i0 < nkt; i0 += 16) {
        uint32_t ba[16], bb[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const bool in = i0 + j < nkt;
          ba[j] = (in && grow < M) ? __float_as_uint(sa_row[i0 + j]) : 0u;
          bb[j] = in ? __float_as_uint(g.sb[sb_row + kt0 + i0 + j]) : 0x3f800000u;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (i0 + j < nkt) {
            pow2 = pow2 && !((ba[j] | bb[j]) & 0x807fffffu);
            const int e = grow < M ? (int)(ba[j] >> 23) + (int)(bb[j] >> 23) - 127 : 0;
            blk[(i0 + j) * 128] = (uint32_t)min(max(e, 0), 254) * 0x01010101u;
          }
        }
      }
      reinterpret_cast<uint32_t*>(sf_all)[nkt * 128 + row] = 0x7f7f7f7fu;
      if (!pow2) dsv4_set_error(DSV4_ERR_BAD_INDEX, 41, grow);  // a scale that is not a power of two
      fence_proxy_async_smem();
      mbar_arrive(&tempty[0]);
    }
    if (nkt > 0) {
      ok = mbar_wait<64>(&tfull[0], 0, abort_flag, 4);
      tc_fence_after();
      if (ok) {
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(lane_addr + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[c * 32 + j] = __uint_as_float(r[j]);
        }
      }
    }
    bool write_out = ok;
    if (g.cluster) {
      // park this split's fp32 partial in shared memory (the pipeline stages are idle by now); the cluster reduces
      // it below.  Rows are padded by 4 floats so that both the row-wise writes here and the 16-byte reads of the
      // reduction are free of bank conflicts.
      float* red = reinterpret_cast<float*>(tiles) + (size_t)row * (BN + 4);
#pragma unroll
      for (int j = 0; j < BN; j += 4)
        *reinterpret_cast<float4*>(red + j) =
            ok ? make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]) : make_float4(0.f, 0.f, 0.f, 0.f);
      write_out = false;
    } else if (g.splits > 1 && g.partial_stride == 0) {
      // publish this split's fp32 partial, the last split to arrive reduces all of them in split order
      const int tile = (batch * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
      float* wsp = g.ws + (((size_t)tile * g.splits + split) * kBM + row) * BN;
#pragma unroll
      for (int j = 0; j < BN; j += 4)
        *reinterpret_cast<float4*>(wsp + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (warp == 2 && lane == 0) *sh_flag = (atomicAdd(&g.counters[tile], 1) == g.splits - 1) ? 1 : 0;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      write_out = write_out && (*sh_flag != 0);
      if (write_out) {
        __threadfence();
#pragma unroll
        for (int j = 0; j < BN; ++j) acc[j] = 0.f;
        for (int s = 0; s < g.splits; ++s) {
          const float* p = g.ws + (((size_t)tile * g.splits + s) * kBM + row) * BN;
#pragma unroll
          for (int j = 0; j < BN; j += 4) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(p + j));
            acc[j] += v.x, acc[j + 1] += v.y, acc[j + 2] += v.z, acc[j + 3] += v.w;
          }
        }
        if (warp == 2 && lane == 0) g.counters[tile] = 0;
      }
    }
    if (g.sp_mode == 3) {
      // reduce-scatter through the switch: leave the partial tile in this rank's own buffer (row-major [T, N] at the
      // same offset on every rank) and tell the tile's owner; the owner's sp_rs_reduce_kernel then asks the switch
      // for the sum of all ranks' copies of its rows (multimem.ld_reduce), so no partial row crosses NVLink twice
      if constexpr (sizeof(OutT) == 2) {
        const int rpr = g.sp.rows_per_rank;
        const int owner = m0 / rpr;
        if (write_out && grow < M) {
          OutT* dst0 = reinterpret_cast<OutT*>(g.sp.peer[g.sp.rank] + g.sp.rs_off) + (size_t)grow * N;
#pragma unroll
          for (int c = 0; c < BN / 32; ++c) {
            const int col = n0 + c * 32;
            if (col < N) store_row_chunk(dst0 + col, &acc[c * 32], N - col);
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 2 && lane == 0) {
          __threadfence_system();
          if (atomicAdd(&g.sp_counters[blockIdx.y], 1) == (int)gridDim.x - 1) {
            g.sp_counters[blockIdx.y] = 0;
            __threadfence_system();
            st_relaxed_sys(sp_flag(g.sp, owner, kSpRS, g.sp.rank, (m0 - owner * rpr) >> 7), g.sp.seq);
          }
        }
      }
      write_out = false;
    }
    if (g.sp_mode == 2) {
      if constexpr (sizeof(OutT) == 2) {
        const int rpr = g.sp.rows_per_rank;
        const int owner = m0 / rpr;                 // a 128-row tile has one owner (rpr is a multiple of 128)
        // Stage the bf16 tile in shared memory (the pipeline stages are idle by now) and store it row-contiguously:
        // consecutive threads write consecutive 16-byte pieces of a row, so a warp's store is a few 64-128-byte
        // segments instead of 32 pieces 8 KB apart -- over NVLink every separate piece is a packet of its own.
        constexpr int LD = BN + 8;                                   // padded row (elements): conflict-free 16-byte access
        __nv_bfloat16* stg = reinterpret_cast<__nv_bfloat16*>(tiles);
        if (write_out) {
#pragma unroll
          for (int j = 0; j < BN; j += 8) {
            uint4 u;
            __nv_bfloat162* pu = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
            for (int e2 = 0; e2 < 4; ++e2) pu[e2] = __floats2bfloat162_rn(acc[j + 2 * e2], acc[j + 2 * e2 + 1]);
            *reinterpret_cast<uint4*>(stg + (size_t)row * LD + j) = u;
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (write_out) {
          OutT* base = reinterpret_cast<OutT*>(g.sp.peer[owner] + g.sp.rs_off) + (size_t)g.sp.rank * rpr * N;
          constexpr int CPR = BN / 8;                                // 16-byte pieces per tile row
          for (int i = threadIdx.x - 64; i < kBM * CPR; i += 128) {
            const int r = i / CPR, cc = i % CPR, gr = m0 + r, col = n0 + cc * 8;
            if (gr < M && col < N)
              st_bulk16(base + (size_t)(gr - owner * rpr) * N + col,
                        *reinterpret_cast<const uint4*>(stg + (size_t)r * LD + cc * 8));
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 2 && lane == 0) {
          __threadfence_system();
          if (atomicAdd(&g.sp_counters[blockIdx.y], 1) == (int)gridDim.x - 1) {
            g.sp_counters[blockIdx.y] = 0;
            __threadfence_system();
            st_relaxed_sys(sp_flag(g.sp, owner, kSpRS, g.sp.rank, (m0 - owner * rpr) >> 7), g.sp.seq);
          }
        }
      }
      write_out = false;
    }
    if (write_out && grow < M) {
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
        const int col = n0 + c * 32;
        if (col < N) {
          OutT* dst = part + (size_t)grow * ld_part + col;
          if (g.accumulate_out) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col + j < N) acc[c * 32 + j] += (float)dst[j];
          }
          store_row_chunk(dst, &acc[c * 32], N - col);
        }
      }
    }
    if (fused && !g.deposit_only) {
      if constexpr (sizeof(OutT) == 2) {
        const int slot = blockIdx.y * gridDim.x + blockIdx.x;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 2 && lane == 0) {
          comm_publish(comm, slot, epoch);
          *sh_flag = comm_wait(comm, slot, epoch) ? 1 : 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (*sh_flag && grow < M) {
#pragma unroll 1
          for (int c8 = 0; c8 < BN; c8 += 16) {
            const int col = n0 + c8;
            if (col + 8 < N) {
              uint4 o0, o1;
              comm_reduce16x2(comm, epoch & 1, (size_t)grow * N + col, (size_t)grow * N + col + 8, o0, o1);
              *reinterpret_cast<uint4*>(out + (size_t)grow * g.ldo + col) = o0;
              *reinterpret_cast<uint4*>(out + (size_t)grow * g.ldo + col + 8) = o1;
            } else if (col < N) {
              *reinterpret_cast<uint4*>(out + (size_t)grow * g.ldo + col) =
                  comm_reduce16(comm, epoch & 1, (size_t)grow * N + col);
            }
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 2 && lane == 0) comm_finish(comm, gridDim.x * gridDim.y);
      }
    }
  }
  if (g.cluster) {
    // Cluster split-K: CTA r of the cluster owns rows [r * 128 / S, (r + 1) * 128 / S) of the tile and adds the S
    // partials in split order (bit-reproducible), reading its peers' shared memory directly.
    const int S2 = g.splits;
    __syncwarp();
    cluster_sync_all();
    if (warp >= 2) {
      const int t = threadIdx.x - 64;                    // 0..127
      const int rows_per = kBM / S2;                     // S2 in {2, 4, 8}
      const int f4_per_row = BN / 4;
      const int total_f4 = rows_per * f4_per_row;
      const uint32_t my_rank = cluster_ctarank();
      const uint32_t red_base = smem_u32(tiles);
      OutT* outb = out + (size_t)batch * g.out_col_pb;
      for (int f = t; f < total_f4; f += 128) {
        const int row = (int)my_rank * rows_per + f / f4_per_row, c4 = f % f4_per_row;
        const uint32_t addr = red_base + (uint32_t)(row * (BN + 4) + c4 * 4) * 4u;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int sp = 0; sp < S2; ++sp) {
          const float4 v = ld_dsmem_f4(addr, (uint32_t)sp);
          a.x += v.x, a.y += v.y, a.z += v.z, a.w += v.w;
        }
        const int grow = m0 + row, col = n0 + c4 * 4;
        if (grow < M && col < N) {
          OutT* dst = outb + (size_t)grow * g.ldo + col;
          float v4[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (col + j < N) {
              if (g.accumulate_out) v4[j] += (float)dst[j];
              dst[j] = (OutT)v4[j];
            }
        }
      }
    }
    cluster_sync_all();  // nobody leaves while a peer may still read its shared memory
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

struct LaunchOpts {
  int batches = 1, a_col_pb = 0, b_row_pb = 0, out_col_pb = 0;
  int splits = 1;
  float* ws = nullptr;
  long long partial_stride = 0;
  int cluster = 0;
  int deposit_only = 0;
  int* counters = nullptr;
  int a_cols = 0, b_rows = 0;  // full extents of the operands (0 = K / N)
  int sb_ld = 0;
  const CommCtx* comm = nullptr;
  int sp_mode = 0;
  const SpCtx* sp = nullptr;
  int* sp_counters = nullptr;
};

int g_weight_prefetch = 0;  // set by dsv4_gemm_set_weight_prefetch

template <int BN, bool FP8, typename OutT>
int launch_gemm(const void* x, const void* w, OutT* out, int M, int N, int K, int ldx, int ldw, int ldo, const float* sa,
                const float* sb, int accumulate_out, cudaStream_t stream, const LaunchOpts& o) {
  using Cfg = GemmCfg<BN, FP8>;
  constexpr int BK = FP8 ? 128 : 64;
  const int esz = FP8 ? 1 : 2;
  if (FP8 && ((K + BK - 1) / BK + o.splits - 1) / o.splits > kMaxKt) return 108;  // scale blocks of one CTA's K range
  CUtensorMap tmA, tmB;
  const uint64_t a_cols = o.a_cols ? o.a_cols : K, b_rows = o.b_rows ? o.b_rows : N;
  if (dsv4_make_tmap_2d(&tmA, x, FP8 ? 0 : 1, a_cols, (uint64_t)M, (uint64_t)ldx * esz, BK, kBM, 3)) return 101;
  if (dsv4_make_tmap_2d(&tmB, w, FP8 ? 0 : 1, (uint64_t)K, b_rows, (uint64_t)ldw * esz, BK, BN, 3)) return 102;
  auto kern = gemm_tn_kernel<BN, FP8, OutT>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return 103;
    attr_set = true;
  }
  dim3 grid((N + BN - 1) / BN, (M + kBM - 1) / kBM, o.batches * o.splits);
  CommCtx comm{};
  if (o.comm) {
    comm = *o.comm;
    // the fused epilogue uses the tile number as its flag slot; a deposit-only launch raises no flags
    if (o.splits != 1 || o.batches != 1) return 104;
    if (!o.deposit_only && (long long)grid.x * grid.y > kCommSlots) return 104;
  }
  GemmArgs g{M, N, K, ldo, sa, sb, o.sb_ld ? o.sb_ld : (K + 127) / 128, accumulate_out, o.a_col_pb, o.b_row_pb,
             o.out_col_pb, o.splits, o.ws, o.counters, o.deposit_only, g_weight_prefetch, o.cluster, o.partial_stride,
             o.sp_mode, o.sp_counters, o.sp ? *o.sp : SpCtx{}};
  if (o.sp_mode && (!o.sp || o.sp->rows_per_rank % kBM || o.batches != 1)) return 106;
  if (o.sp_mode >= 2 && (o.splits != 1 || !o.sp_counters)) return 107;
  if (o.cluster) {
    if (o.splits != 2 && o.splits != 4 && o.splits != 8) return 105;
    dsv4_launch_cluster(kern, grid, 192, Cfg::kSmemBytes, stream, o.splits, tmA, tmB, out, g, comm);
  } else {
    dsv4_launch(kern, grid, 192, Cfg::kSmemBytes, stream, tmA, tmB, out, g, comm);
  }
  return (int)cudaGetLastError();
}

template <bool FP8, typename OutT>
int dispatch_bn(const void* x, const void* w, OutT* out, int M, int N, int K, int ldx, int ldw, int ldo, const float* sa,
                const float* sb, int acc, int bn, cudaStream_t st, const LaunchOpts& o = LaunchOpts{}) {
  if (bn == 0) {
    const int mt = (M + kBM - 1) / kBM * o.batches;
    if (mt * ((N + 127) / 128) >= 98)
      bn = 128;
    else if (mt * ((N + 63) / 64) >= 98)
      bn = 64;
    else
      bn = 32;
  }
  // fused all-reduce epilogue: one flag slot per tile, so a tile count beyond the slots needs the wider tile
  if (o.comm && !o.deposit_only && bn < 64 &&
      (long long)((N + bn - 1) / bn) * ((M + kBM - 1) / kBM) > kCommSlots)
    bn = 64;
  switch (bn) {
    case 128:
      return launch_gemm<128, FP8, OutT>(x, w, out, M, N, K, ldx, ldw, ldo, sa, sb, acc, st, o);
    case 64:
      return launch_gemm<64, FP8, OutT>(x, w, out, M, N, K, ldx, ldw, ldo, sa, sb, acc, st, o);
    default:
      return launch_gemm<32, FP8, OutT>(x, w, out, M, N, K, ldx, ldw, ldo, sa, sb, acc, st, o);
  }
}

}  // namespace

// on != 0: the callers promise that the weight operand (w) of every GEMM launched from now on is not produced by the
// kernel that precedes it in the stream (model weights are static), so its first tiles may be fetched before the
// dependent-launch wait.  Off by default.
DSV4_API int dsv4_gemm_set_weight_prefetch(int on) {
  g_weight_prefetch = on ? 1 : 0;
  return 0;
}

// Workspace floats needed for a split-K launch: tiles * splits * 128 * bn.
DSV4_API long long dsv4_gemm_splitk_ws_elems(int M, int N, int bn, int batches, int splits) {
  const long long tiles = (long long)((N + bn - 1) / bn) * ((M + kBM - 1) / kBM) * batches;
  return tiles * splits * kBM * bn;
}

// out dtype: 0 = bf16, 1 = fp32.  ld* are row strides in elements.  bn = 0 picks the tile width.
// batches > 1: batch b uses A columns [b*K, (b+1)*K) of x (ldx covers all batches), W rows [b*N, (b+1)*N) and output
// columns [b*N, (b+1)*N).  splits > 1 needs ws (dsv4_gemm_splitk_ws_elems floats) and counters (>= tiles ints, zero).
DSV4_API int dsv4_gemm_bf16(const void* x, const void* w, void* out, int M, int N, int K, int ldx, int ldw, int ldo,
                            int out_fp32, int accumulate_out, int bn, int batches, int splits, float* ws, int* counters,
                            cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((K % 8) || (ldx % 8) || (ldw % 8)) return 110;
  LaunchOpts o;
  o.batches = batches < 1 ? 1 : batches;
  o.splits = splits < 1 ? 1 : splits;
  o.ws = ws, o.counters = counters;
  if (o.batches > 1) o.a_col_pb = K, o.b_row_pb = N, o.out_col_pb = N, o.a_cols = K * o.batches, o.b_rows = N * o.batches;
  if (o.splits > 1 && bn == 0) return 116;
  if (o.splits > 1 && (!ws || !counters)) o.cluster = 1;  // no workspace given: reduce inside a thread-block cluster
  if (out_fp32)
    return dispatch_bn<false, float>(x, w, (float*)out, M, N, K, ldx, ldw, ldo, nullptr, nullptr, accumulate_out, bn,
                                     stream, o);
  return dispatch_bn<false, __nv_bfloat16>(x, w, (__nv_bfloat16*)out, M, N, K, ldx, ldw, ldo, nullptr, nullptr,
                                           accumulate_out, bn, stream, o);
}

// Split-K without the reduction: split s writes x[:, K_s] . w[:, K_s]^T as fp32 to out + s * split_stride (row stride
// ldo); the consuming kernel adds the `splits` partial products in order.  For very skinny outputs (a handful of
// columns over a long K) this spreads both the weight stream and the reduction over the GPU.
DSV4_API int dsv4_gemm_bf16_partials(const void* x, const void* w, float* out, int M, int N, int K, int ldx, int ldw,
                                     int ldo, int bn, int splits, long long split_stride, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((K % 8) || (ldx % 8) || (ldw % 8) || splits < 1 || split_stride < (long long)M * ldo) return 118;
  LaunchOpts o;
  o.splits = splits;
  o.partial_stride = split_stride;
  return dispatch_bn<false, float>(x, w, out, M, N, K, ldx, ldw, ldo, nullptr, nullptr, 0, bn ? bn : 32, stream, o);
}

// x: e4m3 [M,K] with sa fp32 [M, K/128];  w: e4m3 [N,K] with sb fp32 [ceil(N/128), K/128].
DSV4_API int dsv4_gemm_fp8(const void* x, const void* w, void* out, const float* sa, const float* sb, int M, int N, int K,
                           int ldx, int ldw, int ldo, int out_fp32, int accumulate_out, int bn, int splits, float* ws,
                           int* counters, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((K % 128) || (ldx % 16) || (ldw % 16)) return 111;
  LaunchOpts o;
  o.splits = splits < 1 ? 1 : splits;
  o.ws = ws, o.counters = counters;
  if (o.splits > 1 && bn == 0) return 117;
  if (o.splits > 1 && (!ws || !counters)) o.cluster = 1;
  if (out_fp32)
    return dispatch_bn<true, float>(x, w, (float*)out, M, N, K, ldx, ldw, ldo, sa, sb, accumulate_out, bn, stream, o);
  return dispatch_bn<true, __nv_bfloat16>(x, w, (__nv_bfloat16*)out, M, N, K, ldx, ldw, ldo, sa, sb, accumulate_out, bn,
                                          stream, o);
}

// Row-sharded exchange, consumer side ("all-gather -> projection"): x / sa are this rank's gathered buffer; the
// producer warp of every CTA waits for the owner's flag of its 128-row block before it loads the block's A tiles.
// partials != 0: split-K partial products like dsv4_gemm_bf16_partials (bf16 operands only).
DSV4_API int dsv4_gemm_fp8_gated(const void* x, const void* w, void* out, const float* sa, const float* sb, int M, int N,
                                 int K, int ldx, int ldw, int ldo, int bn, const SpCtx* sp, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((K % 128) || (ldx % 16) || (ldw % 16)) return 111;
  LaunchOpts o;
  o.sp_mode = 1;
  o.sp = sp;
  return dispatch_bn<true, __nv_bfloat16>(x, w, (__nv_bfloat16*)out, M, N, K, ldx, ldw, ldo, sa, sb, 0, bn, stream, o);
}
DSV4_API int dsv4_gemm_bf16_partials_gated(const void* x, const void* w, float* out, int M, int N, int K, int ldx,
                                           int ldw, int ldo, int bn, int splits, long long split_stride,
                                           const SpCtx* sp, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((K % 8) || (ldx % 8) || (ldw % 8) || splits < 1 || split_stride < (long long)M * ldo) return 118;
  LaunchOpts o;
  o.splits = splits;
  o.partial_stride = split_stride;
  o.sp_mode = 1;
  o.sp = sp;
  return dispatch_bn<false, float>(x, w, out, M, N, K, ldx, ldw, ldo, nullptr, nullptr, 0, bn ? bn : 32, stream, o);
}
// Row-sharded exchange, producer side ("projection -> reduce-scatter"): the epilogue stores every partial row into its
// owner's buffer over NVLink; dsv4_sp_rs_reduce on the owner adds the partials.  counters: >= ceil(M / 128) zero ints.
DSV4_API int dsv4_gemm_fp8_rs(const void* x, const void* w, const float* sa, const float* sb, int M, int N, int K,
                              int ldx, int ldw, int bn, const SpCtx* sp, int* counters, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((K % 128) || (ldx % 16) || (ldw % 16) || (N % 8) || N != sp->hidden) return 112;
  LaunchOpts o;
  o.sp_mode = (sp->use_mc && sp->mc) ? 3 : 2;   // in-switch reduction where a multicast mapping exists
  o.sp = sp;
  o.sp_counters = counters;
  return dispatch_bn<true, __nv_bfloat16>(x, w, (__nv_bfloat16*)nullptr, M, N, K, ldx, ldw, N, sa, sb, 0, bn, stream, o);
}

// Fused projection + all-reduce: every rank multiplies its K-shard, the epilogue publishes the partial tile to the
// rank's symmetric buffer and reduces the peers' tiles over NVLink (see comm.cuh).  out is bf16 [M,N], dense.
// deposit != 0: the GEMM only leaves its partial product in the channel's symmetric buffer (out is not written);
// dsv4_allreduce(x = null, ...) on the same channel must follow.  For small row counts this beats reducing in the
// GEMM epilogue, whose 128 x 32 tiles make the peer reads 64-byte pieces.
DSV4_API int dsv4_gemm_fp8_allreduce(const void* x, const void* w, void* out, const float* sa, const float* sb, int M,
                                     int N, int K, int ldx, int ldw, const CommCtx* comm, int bn, int deposit,
                                     cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((K % 128) || (ldx % 16) || (ldw % 16) || (N % 8)) return 112;
  if ((long long)M * N * 2 > comm->data_bytes) return 113;
  LaunchOpts o;
  o.comm = comm;
  o.deposit_only = deposit ? 1 : 0;
  return dispatch_bn<true, __nv_bfloat16>(x, w, (__nv_bfloat16*)out, M, N, K, ldx, ldw, N, sa, sb, 0, bn, stream, o);
}
DSV4_API int dsv4_gemm_bf16_allreduce(const void* x, const void* w, void* out, int M, int N, int K, int ldx, int ldw,
                                      const CommCtx* comm, int bn, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((K % 8) || (ldx % 8) || (ldw % 8) || (N % 8)) return 114;
  if ((long long)M * N * 2 > comm->data_bytes) return 115;
  LaunchOpts o;
  o.comm = comm;
  return dispatch_bn<false, __nv_bfloat16>(x, w, (__nv_bfloat16*)out, M, N, K, ldx, ldw, N, nullptr, nullptr, 0, bn,
                                           stream, o);
}
