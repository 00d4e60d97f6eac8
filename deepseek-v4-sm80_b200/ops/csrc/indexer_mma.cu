// Sparse-attention indexer logits on the 5th-generation tensor cores.
//
//   logits[t, j] = k_scale[row_j] * sum_h relu(q[t,h,:] . k[row_j,:]) * w[t,h]     for j < (pos[t]+1)/4, else -inf
//
// q [T, 64, 128] and k [rows, 128] are e4m3 codes, so the contraction is one FP8 GEMM per (request, token group):
//   D[128 keys, 64 heads x G tokens] = K_tile[128 keys, 128] . Q_group[64 x G, 128]^T      (tcgen05.mma kind::f8f6f4)
// with the KEY rows on the 128 tensor-memory lanes and the heads of up to four consecutive tokens of the same request
// on the N dimension.  The reduction over heads is then a per-lane sum over 64 accumulator columns: the epilogue
// thread that owns a lane reads its columns with tcgen05.ld, applies relu and the folded per-head weight, multiplies
// by the key's scale and writes one logit per token -- no cross-lane traffic at all.  (The reference computes the
// same logits with tl.dot: python/minisgl/kernel/triton/deepseek_v4.py:1296-1384.)
//
// A CTA owns one token group and a stride of the request's 128-key blocks.  Warp 0 walks the page table and feeds a
// ring of key tiles by TMA (a page's compressed rows are contiguous, so a tile is 128 / rows-per-box box copies),
// warp 1 issues the MMAs into one of two accumulators, warps 2-5 are the epilogue (one TMEM lane quarter each).
// Tokens of one group that belong to different requests (decode batches, request boundaries inside a prefill chunk)
// are handled as separate passes over their own keys with N = 64.  Every wait is bounded.
#include "common.cuh"

namespace {

constexpr int DI = 128;          // indexer head dim = bytes per e4m3 row = one 128-byte swizzle span
constexpr int HEADS = 64;
constexpr int KB = 128;          // keys per tile (TMEM lanes)
constexpr int TGMAX = 4;         // tokens per group (N = 256 at most)
constexpr int SA = 6;            // key-tile ring (four-token groups); one-token groups use 4 stages
constexpr int kATile = KB * DI;  // 16 KiB
constexpr int kQTile = HEADS * DI;  // 8 KiB per token

struct IdxArgs {
  const float* wf;        // [T, 64] folded head weights
  const float* kscale;    // [rows]
  const int* slots;       // [T]
  const int* pos;         // [T]
  const int* page_table;  // [slots, ld_pt] token locations
  int ld_pt;
  int ps;                 // page size in tokens
  float* logits;          // [T, width]
  int width;
  int T;
  int tg;                 // tokens per group (1, 2 or 4)
  int box_rows;           // key rows per TMA box = min(ps / 4, 64)
  int stages;             // key-tile ring depth
  int tmem_cols;          // tensor-memory columns: two accumulators of tg * 64 columns, rounded to a power of two
};
// Shared memory and tensor memory are sized by the group width: a decode launch (one token per group, N = 64) then
// fits three CTAs on an SM instead of one, which is what hides the page-table -> TMA -> MMA latency chain there.
inline int idx_smem_bytes(int tg, int stages) { return stages * kATile + tg * kQTile + tg * HEADS * 4 + 256 + 1024; }

constexpr int kSmemBytes = SA * kATile + TGMAX * kQTile + TGMAX * HEADS * 4 + 256 + 1024;

__global__ void __launch_bounds__(192, 1)
indexer_logits_mma_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmQ,
                          const IdxArgs a) {
  extern __shared__ uint8_t ix_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(ix_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* atiles = smem;                                   // [SA][128 keys][128 B], 128B-swizzled by TMA
  const int NS = a.stages;
  uint8_t* qtile = smem + NS * kATile;                      // [tg * 64 rows][128 B]
  float* wfs = reinterpret_cast<float*>(qtile + a.tg * kQTile);   // [tg][64]
  uint64_t* full = reinterpret_cast<uint64_t*>(wfs + a.tg * HEADS);
  uint64_t* empty = full + SA;
  uint64_t* tfull = empty + SA;    // [2]
  uint64_t* tempty = tfull + 2;    // [2]
  uint64_t* qfull = tempty + 2;    // [1]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(qfull + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = blockIdx.y * a.tg;
  const int ng = min(a.tg, a.T - t0);          // tokens of this group
  const int split = blockIdx.x, nsplit = gridDim.x;
  const int rpp = a.ps >> 2;                   // compressed rows per page

  if (threadIdx.x == 0) {
    for (int i = 0; i < NS; ++i) mbar_init(&full[i], 1), mbar_init(&empty[i], 1);
    for (int i = 0; i < 2; ++i) mbar_init(&tfull[i], 1), mbar_init(&tempty[i], 128);
    mbar_init(qfull, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmQ);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, (uint32_t)a.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  pdl_wait();
  pdl_launch_dependents();  // only after the own wait (common.cuh: programmatic dependent launch)

  // passes: maximal runs of consecutive tokens of the group that share a request slot (at most 4 runs)
  int p_first[TGMAX], p_cnt[TGMAX], p_blocks[TGMAX], p_slot[TGMAX], npass = 0;
  int n_tok[TGMAX];
  for (int g = 0; g < TGMAX; ++g) n_tok[g] = 0;
  for (int g = 0; g < ng; ++g) {
    const int sl = a.slots[t0 + g];
    n_tok[g] = min((a.pos[t0 + g] + 1) >> 2, a.width);
    if (npass > 0 && p_slot[npass - 1] == sl) {
      p_cnt[npass - 1]++;
    } else {
      p_first[npass] = g, p_cnt[npass] = 1, p_slot[npass] = sl;
      npass++;
    }
  }
  for (int p = 0; p < npass; ++p) {
    int nmax = 0;
    for (int g = p_first[p]; g < p_first[p] + p_cnt[p]; ++g) nmax = max(nmax, n_tok[g]);
    p_blocks[p] = (nmax + KB - 1) / KB;
  }
  // columns past the last computed block of each token are -inf (all threads, blocks strided like the work)
  {
    const int wblocks = (a.width + KB - 1) / KB;
    for (int p = 0; p < npass; ++p)
      for (int g = p_first[p]; g < p_first[p] + p_cnt[p]; ++g)
        for (int kb = p_blocks[p] + split; kb < wblocks; kb += nsplit)
          for (int j = kb * KB + threadIdx.x; j < min(kb * KB + KB, a.width); j += blockDim.x)
            a.logits[(size_t)(t0 + g) * a.width + j] = -INFINITY;
  }

  if (warp == 0) {
    // ---------------- producer: Q tile once, then key tiles through the ring
    if (lane == 0) {
      mbar_expect_tx(qfull, (uint32_t)ng * kQTile);
      for (int g = 0; g < ng; ++g) tma_load_2d(qtile + g * kQTile, &tmQ, qfull, 0, (t0 + g) * HEADS);
    }
    const int nloads = KB / a.box_rows;        // boxes per key tile (2 for 256-token pages), one per lane
    int it = 0;
    bool dead = false;
    for (int p = 0; p < npass && !dead; ++p) {
      const int* pt = a.page_table + (size_t)p_slot[p] * a.ld_pt;
      int nmax = 0;
      for (int g = p_first[p]; g < p_first[p] + p_cnt[p]; ++g) nmax = max(nmax, n_tok[g]);
      for (int kb = split; kb < p_blocks[p]; kb += nsplit, ++it) {
        const int s = it % NS;
        // each lane resolves the rows of its boxes before the stage wait, so the lookups overlap the wait
        int rowsrc[4];
        int mine = 0;
        for (int h = lane, u = 0; h < nloads && u < 4; h += 32, ++u) {
          const int j = kb * KB + h * a.box_rows;
          rowsrc[u] = -1;
          if (j < nmax) {
            const int loc = pt[4 * j + 3];
            rowsrc[u] = (loc / a.ps) * rpp + (loc % a.ps) / 4;
            ++mine;
          }
        }
        int total = mine;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
        int ok = 1;
        if (lane == 0) {
          ok = mbar_wait<32>(&empty[s], ((it / NS) & 1) ^ 1, abort_flag, 11) ? 1 : 0;
          if (ok) mbar_expect_tx(&full[s], (uint32_t)total * a.box_rows * DI);
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) {
          dead = true;
          break;
        }
        for (int h = lane, u = 0; h < nloads && u < 4; h += 32, ++u)
          if (rowsrc[u] >= 0)
            tma_load_2d(atiles + s * kATile + h * a.box_rows * DI, &tmK, &full[s], 0, rowsrc[u]);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer
    if (lane == 0) {
      bool ok = mbar_wait(qfull, 0, abort_flag, 12);
      int it = 0;
      for (int p = 0; p < npass && ok; ++p) {
        const uint32_t idesc = umma_idesc(KB, HEADS * p_cnt[p], 0, 0);
        const uint8_t* qb = qtile + p_first[p] * kQTile;
        for (int kb = split; kb < p_blocks[p]; kb += nsplit, ++it) {
          const int s = it % NS, b = it & 1;
          if (!mbar_wait(&tempty[b], ((it >> 1) & 1) ^ 1, abort_flag, 13)) {
            ok = false;
            break;
          }
          if (!mbar_wait(&full[s], (it / NS) & 1, abort_flag, 14)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t d = tmem_base + b * (a.tg * HEADS);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f8(d, umma_desc_k128(atiles + s * kATile, k * 32), umma_desc_k128(qb, k * 32), idesc, k > 0);
          umma_commit(&empty[s]);
          umma_commit(&tfull[b]);
        }
      }
    }
  } else {
    // ---------------- epilogue: warp w owns TMEM lanes (w % 4) * 32 .. + 31, i.e. 32 keys of every tile
    const int q = warp & 3;
    const int key_in_tile = q * 32 + lane;
    for (int i = threadIdx.x - 64; i < ng * HEADS; i += 128) wfs[i] = a.wf[(size_t)t0 * HEADS + i];
    asm volatile("bar.sync 1, 128;" ::: "memory");
    int it = 0;
    bool ok = true;
    for (int p = 0; p < npass && ok; ++p) {
      const int* pt = a.page_table + (size_t)p_slot[p] * a.ld_pt;
      int nmax = 0;
      for (int g = p_first[p]; g < p_first[p] + p_cnt[p]; ++g) nmax = max(nmax, n_tok[g]);
      for (int kb = split; kb < p_blocks[p]; kb += nsplit, ++it) {
        const int b = it & 1;
        const int j = kb * KB + key_in_tile;
        float ks = 0.f;
        if (j < nmax) {   // resolved while the tile is still being multiplied
          const int loc = pt[4 * j + 3];
          ks = a.kscale[(size_t)(loc / a.ps) * rpp + (loc % a.ps) / 4];
        }
        if (!mbar_wait<64>(&tfull[b], (it >> 1) & 1, abort_flag, 15)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + b * (a.tg * HEADS);
        for (int c = 0; c < p_cnt[p]; ++c) {
          const int g = p_first[p] + c;
          const float* w = wfs + g * HEADS;
          float acc = 0.f;
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            uint32_t r[32];
            tmem_ld_32x32(taddr + c * HEADS + half * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int h = 0; h < 32; ++h) acc = fmaf(fmaxf(__uint_as_float(r[h]), 0.f), w[half * 32 + h], acc);
          }
          if (j < a.width) a.logits[(size_t)(t0 + g) * a.width + j] = j < n_tok[g] ? acc * ks : -INFINITY;
        }
        tc_fence_before();
        mbar_arrive(&tempty[b]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, (uint32_t)a.tmem_cols);
}

}  // namespace

int dsv4_make_tmap_2d(CUtensorMap* out, const void* base, int elem, uint64_t inner, uint64_t outer,
                      uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, int swizzle);

// qc u8 [T, 64, 128], wf fp32 [T, 64], kvals u8 [krows, 128], kscale fp32 [krows]; logits fp32 [T, width].
// Supported: 64 heads of 128 dims, page size >= 32 tokens with ps / 4 dividing 64 or a multiple of 64 (the callers
// keep the CUDA-core kernel of indexer.cu for anything else).
// tg: tokens per group (1: decode batches, 4: prefill chunks with long runs per request); nsplit: CTAs per group.
DSV4_API int dsv4_indexer_logits_mma(const void* qc, const float* wf, const void* kvals, const float* kscale,
                                     long long krows, const int* slots, const int* pos, const int* page_table,
                                     int ld_pt, int ps, float* logits, int width, int t, int heads, int d, int tg,
                                     int nsplit, cudaStream_t st) {
  if (t <= 0 || width <= 0) return 0;
  if (heads != HEADS || d != DI) return 470;
  const int rpp = ps / 4;
  if (ps % 4 || rpp <= 0 || !((rpp <= 64 && 64 % rpp == 0) || rpp % 64 == 0)) return 471;
  if (tg != 1 && tg != 2 && tg != 4) return 472;
  const int box_rows = rpp < 64 ? rpp : 64;
  // every box must start on a 1024-byte boundary of its tile so that all boxes share one 128-byte swizzle pattern
  if (box_rows < 8) return 473;
  CUtensorMap tmK, tmQ;
  if (dsv4_make_tmap_2d(&tmK, kvals, 0, DI, (uint64_t)krows, DI, DI, box_rows, 3)) return 474;
  if (dsv4_make_tmap_2d(&tmQ, qc, 0, DI, (uint64_t)t * HEADS, DI, DI, HEADS, 3)) return 475;
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(indexer_logits_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) !=
        cudaSuccess)
      return 476;
    set = true;
  }
  const int stages = tg == 1 ? 4 : SA;
  const int tmem_cols = tg == 1 ? 128 : tg == 2 ? 256 : 512;
  IdxArgs a{wf, kscale, slots, pos, page_table, ld_pt, ps, logits, width, t, tg, box_rows, stages, tmem_cols};
  const int groups = (t + tg - 1) / tg;
  if (nsplit < 1) nsplit = 1;
  dsv4_launch(indexer_logits_mma_kernel, dim3(nsplit, groups), 192, idx_smem_bytes(tg, stages), st, tmK, tmQ, a);
  return (int)cudaGetLastError();
}
