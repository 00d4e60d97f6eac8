// Sparse MQA attention over the paged caches: per token, all local heads attend
//   {sink} U {selected C4 rows | all C128 rows | nothing} U {sliding window rows},
// keys and values being the same 512-d latent row (K = V), softmax scale 512^-1/2.
//
// One CTA per token.  Every gathered row is fetched once (cp.async into 128B-swizzled shared memory, double
// buffered) and shared by all local heads; both contractions run on the tensor cores with warp-level
// mma.sync.m16n8k16 (bf16 in, fp32 accumulate): with 8..64 heads per token the M extent is 16..64, far below the
// 128-row tiles tcgen05 wants, and the kernel is bound by the row gather, so the warp-level shape is the better fit.
//   S phase : warp (mt, g) computes the 16 x 8 score tile of head tile mt and key group g (32 k-steps)
//   softmax : online (m, l) per head, probabilities to shared memory as bf16
//   PV phase: warp (mt, g) owns head tile mt and a 512/G slice of the output dims in registers
// The kernel walks the request's page-table row itself, so no index surface is materialised: compressed entry j of
// ratio r lives at row comp_row(page_table[slot, j*r + r-1]); window position p lives at
// swa_map[loc / ps] * ps + loc % ps.  (m, l) start at (sink, 1), which adds exp(sink - m) to the denominator only --
// the reference's two-source kernel semantics
// (python/minisgl/kernel/csrc/jit/dsv4_sparse_attention_two_source_bf16.cu:77-168).
//
// Split-KV (decode with few tokens and long histories): grid.y CTAs share one token, each takes a contiguous range of
// the token's key tiles and leaves its unnormalised accumulator with its running (max, sum) in a scratch buffer; the
// last CTA of the token to finish (a per-token counter) merges the partials in split order --
//   M = max_s m_s,  L = sum_s l_s e^(m_s - M),  o = sum_s acc_s e^(m_s - M) / L
// -- and runs the usual epilogue.  The sink belongs to split 0.  The reference's decode kernel splits the same way
// (python/minisgl/kernel/triton/deepseek_v4.py:1645, :2002-2050, up to 16 splits).
#include "common.cuh"
#include "rope.cuh"

namespace {

constexpr int D = 512;

__device__ __forceinline__ void cp_async16_zfill(void* smem, const void* g, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem)), "l"(g), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

struct AttnArgs {
  const __nv_bfloat16* q;
  __nv_bfloat16* o;
  const int* slots;
  const int* pos;
  const int* page_table;
  int ld_pt;
  const __nv_bfloat16* swa;
  const int* swa_map;
  const __nv_bfloat16* comp;
  const int* topk_idx;
  const int* topk_len;
  int topk_width;
  int mode;   // 0: window only, 1: compressed entries from topk_idx, 2: all compressed entries
  int ratio;
  const float* sink;
  float scale;
  int ps;
  int window;
  const int* num_valid;
  int out_rope;   // != 0: rotate the last rp.rotary_dim dims of every output head row by -position (the inverse
  RopeParams rp;  //       RoPE the output projection expects), on the bf16-rounded values, in the epilogue
  int nsplit;        // CTAs per token (grid.y); > 1 needs the three buffers below
  float* part_acc;   // [t][nsplit][HL][512] unnormalised accumulators
  float* part_ml;    // [t][nsplit][HL][2]   running max and sum
  int* counters;     // [t] zero between launches
};

// row of 512 bf16 = 64 chunks of 16 B; chunk c of row r is stored at chunk (c ^ (r & 7))
__device__ __forceinline__ int swz_row(int r, int c) { return (c & ~7) | ((c ^ r) & 7); }

template <int HL>
struct AttnCfg {
  static constexpr int HP = HL < 16 ? 16 : HL;          // padded head rows
  static constexpr int MT = HP / 16;                     // 16-row head tiles
  static constexpr int NW = MT >= 4 ? 16 : 8;            // warps
  static constexpr int G = NW / MT;                      // warps per head tile
  static constexpr int KT = 8 * G;                       // keys per tile: one 16x8 score tile per warp
  static constexpr int DW = D / G;                       // output dims per warp
  static constexpr int NT = DW / 8;                      // output n-tiles per warp
  static constexpr int TPR = NW * 32 / HP;               // softmax threads per head row
  static constexpr int PCH = KT / 8;                     // 16-byte chunks per probability row
  static constexpr int RB = 1024;                        // keys whose rows are resolved per pass (multiple of KT)
  static constexpr int SMEM =
      HP * D * 2 + 2 * KT * D * 2 + HP * KT * 4 + HP * KT * 2 + 3 * HP * 4 + 2 * KT * 4 + RB * 4;
};

template <int HL>
__global__ void __launch_bounds__(AttnCfg<HL>::NW * 32) sparse_attn_kernel(AttnArgs a) {
  pdl_entry();
  using C = AttnCfg<HL>;
  constexpr int HP = C::HP, MT = C::MT, KT = C::KT, NT = C::NT, TPR = C::TPR, PCH = C::PCH;
  constexpr int NTHR = C::NW * 32;
  extern __shared__ __align__(128) uint8_t attn_smem[];
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(attn_smem);   // [HP][D] swizzled
  __nv_bfloat16* kvs = qs + HP * D;                                  // [2][KT][D] swizzled
  float* ss = reinterpret_cast<float*>(kvs + 2 * KT * D);            // [HP][KT] scores
  __nv_bfloat16* pb = reinterpret_cast<__nv_bfloat16*>(ss + HP * KT);  // [HP][KT] probabilities, swizzled
  float* alpha = reinterpret_cast<float*>(pb + HP * KT);             // [HP]
  float* ms = alpha + HP;                                            // [HP]
  float* ls = ms + HP;                                               // [HP]
  int* valid = reinterpret_cast<int*>(ls + HP);                      // [2][KT]
  int* rowsrc = valid + 2 * KT;                                      // [RB] resolved cache row per key, -1: masked
  constexpr int RB = C::RB;
  constexpr int kSwaBit = 1 << 30;                                   // set: row of the window cache, else compressed

  const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int split = blockIdx.y, nsplit = a.nsplit;
  if (a.num_valid && t >= *a.num_valid) {
    if (split == 0)
      for (int i = tid; i < HL * D / 8; i += NTHR)
        reinterpret_cast<uint4*>(a.o + (size_t)t * HL * D)[i] = make_uint4(0, 0, 0, 0);
    return;
  }
  const int p = a.pos[t], slot = a.slots[t];
  const int* pt = a.page_table + (size_t)slot * a.ld_pt;
  int nc = 0;
  if (a.mode == 1) nc = max(a.topk_len[t], 0);
  if (a.mode == 2) nc = (p + 1) / a.ratio;
  const int ns = min(p + 1, a.window);
  const int ntot = nc + ns;
  const int ntiles = (ntot + KT - 1) / KT;
  const int rpp = a.ratio > 0 ? max(a.ps / a.ratio, 1) : 1;

  // Q -> shared (rows >= HL are zero)
  for (int i = tid; i < HP * 64; i += NTHR) {
    const int r = i >> 6, c = i & 63;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < HL) v = reinterpret_cast<const uint4*>(a.q + ((size_t)t * HL + r) * D)[c];
    reinterpret_cast<uint4*>(qs + r * D)[swz_row(r, c)] = v;
  }
  // the sink starts split 0's running (max, sum); the other splits start empty (a finite floor instead of -inf keeps
  // exp(m_old - m_new) well defined for a split that meets no valid key)
  if (tid < HP) {
    if (split == 0)
      ms[tid] = tid < HL ? a.sink[tid] : 0.f, ls[tid] = 1.f;
    else
      ms[tid] = -1e30f, ls[tid] = 0.f;
  }
  // this CTA's keys: a contiguous range of whole tiles
  const int tiles_per = (ntiles + nsplit - 1) / nsplit;
  const int k_lo = min(split * tiles_per * KT, ntot), k_hi = min((split + 1) * tiles_per * KT, ntot);

  // Rows of keys [base, base + RB) -> rowsrc.  A key's row hangs on a chain of two or three dependent loads
  // (selected index -> page-table entry -> window slot); resolving a tile's keys right before its gather would put
  // that chain in front of every tile, so all keys of a pass are resolved together, stage by stage, each thread
  // keeping RB / NTHR independent chains in flight.  A decode token (at most 128 + 512 keys) needs one pass.
  auto resolve = [&](int base) {
    constexpr int PER = RB / NTHR;
    int ppos[PER], loc[PER];
#pragma unroll
    for (int u = 0; u < PER; ++u) {
      const int key = base + tid + u * NTHR;
      ppos[u] = -1;
      if (key < nc) {
        const int j = a.mode == 1 ? a.topk_idx[(size_t)t * a.topk_width + key] : key;
        if (j >= 0) ppos[u] = j * a.ratio + a.ratio - 1;
      } else if (key < ntot) {
        ppos[u] = p - ns + 1 + (key - nc);
      }
    }
#pragma unroll
    for (int u = 0; u < PER; ++u) loc[u] = ppos[u] >= 0 ? pt[ppos[u]] : -1;
#pragma unroll
    for (int u = 0; u < PER; ++u) {
      const int key = base + tid + u * NTHR;
      int e = -1;
      if (loc[u] >= 0) {
        if (key < nc) {
          e = (loc[u] / a.ps) * rpp + (loc[u] % a.ps) / a.ratio;
        } else {
          const int sl = a.swa_map[loc[u] / a.ps];
          if (sl >= 0) e = (sl * a.ps + loc[u] % a.ps) | kSwaBit;
        }
      }
      rowsrc[tid + u * NTHR] = e;
    }
  };

  int rbase = 0;                       // first key whose row sits in rowsrc[0]
  constexpr int TPK = NTHR / KT;       // threads cooperating on one key row
  constexpr int CPT = 64 / TPK;        // 16-byte chunks per thread
  auto issue_tile = [&](int tile, int buf) {
    const int kk = tid / TPK, part = tid % TPK;
    const int e = rowsrc[tile * KT + kk - rbase];
    const __nv_bfloat16* src = nullptr;
    if (e >= 0) src = (e & kSwaBit) ? a.swa + (size_t)(e & (kSwaBit - 1)) * D : a.comp + (size_t)e * D;
    __nv_bfloat16* dst = kvs + ((size_t)buf * KT + kk) * D;
    const __nv_bfloat16* s0 = src ? src : a.swa;
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
      const int ch = part + TPK * c;
      cp_async16_zfill(dst + swz_row(kk, ch) * 8, s0 + ch * 8, src != nullptr);
    }
    if (part == 0) valid[buf * KT + kk] = src != nullptr;
    cp_async_commit();
  };

  const int mt = warp % MT, g = warp / MT;
  float acc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

  for (int base = k_lo; base < k_hi; base += RB) {
  const int tile_lo = base / KT, tile_hi = min((k_hi + KT - 1) / KT, (base + RB) / KT);
  rbase = base;
  resolve(base);
  __syncthreads();
  issue_tile(tile_lo, tile_lo & 1);
  for (int tile = tile_lo; tile < tile_hi; ++tile) {
    const int buf = tile & 1;
    if (tile + 1 < tile_hi) {
      issue_tile(tile + 1, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const __nv_bfloat16* kt = kvs + (size_t)buf * KT * D;
    // ---- S = Q K^T : one 16 x 8 tile per warp (head tile mt, keys g*8 .. g*8+7)
    {
      float s0[4] = {0, 0, 0, 0}, s1[4] = {0, 0, 0, 0};
      const int arow = mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
      const int brow = g * 8 + (lane & 7);
#pragma unroll 4
      for (int ks = 0; ks < 32; ks += 2) {
        uint32_t af[4], af2[4], bf[4];
        ldsm_x4(af, qs + arow * D + swz_row(arow, ks * 2 + (lane >> 4)) * 8);
        ldsm_x4(af2, qs + arow * D + swz_row(arow, ks * 2 + 2 + (lane >> 4)) * 8);
        ldsm_x4(bf, kt + brow * D + swz_row(brow, ks * 2 + (lane >> 3)) * 8);
        mma_bf16(s0, af, bf[0], bf[1]);
        mma_bf16(s1, af2, bf[2], bf[3]);
      }
      const int r0 = mt * 16 + (lane >> 2), c0 = g * 8 + (lane & 3) * 2;
      *reinterpret_cast<float2*>(ss + r0 * KT + c0) = make_float2((s0[0] + s1[0]) * a.scale, (s0[1] + s1[1]) * a.scale);
      *reinterpret_cast<float2*>(ss + (r0 + 8) * KT + c0) =
          make_float2((s0[2] + s1[2]) * a.scale, (s0[3] + s1[3]) * a.scale);
    }
    __syncthreads();
    // ---- online softmax: TPR threads per head row, 4 keys each
    {
      const int row = tid / TPR, seg = tid % TPR;
      float v[4];
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int k = seg * 4 + i;
        v[i] = valid[buf * KT + k] ? ss[row * KT + k] : -INFINITY;
        mx = fmaxf(mx, v[i]);
      }
#pragma unroll
      for (int o = TPR / 2; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float m_old = ms[row];
      const float m_new = fmaxf(m_old, mx);
      float sum = 0.f;
      __nv_bfloat16 pv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float e = __expf(v[i] - m_new);
        pv[i] = f2bf(e);
        sum += bf2f(pv[i]);
      }
#pragma unroll
      for (int o = TPR / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      // 4 keys = 8 bytes = half a 16-byte chunk
      const int ch = seg >> 1, half = seg & 1;
      constexpr int RP = 8 / PCH;  // rows per 128 bytes
      const int pch = ch ^ ((row / RP) % PCH);
      *reinterpret_cast<uint2*>(pb + row * KT + pch * 8 + half * 4) = *reinterpret_cast<uint2*>(pv);
      __syncwarp();
      if (seg == 0) {
        const float al = __expf(m_old - m_new);
        alpha[row] = al;
        ms[row] = m_new;
        ls[row] = ls[row] * al + sum;
      }
    }
    __syncthreads();
    // ---- O += P V : head tile mt, output dims [g*DW, (g+1)*DW)
    {
      const float al0 = alpha[mt * 16 + (lane >> 2)], al1 = alpha[mt * 16 + (lane >> 2) + 8];
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        acc[i][0] *= al0, acc[i][1] *= al0, acc[i][2] *= al1, acc[i][3] *= al1;
      }
      constexpr int RP = 8 / PCH;
      const int prow = mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int kk = 0; kk < KT / 16; ++kk) {
        uint32_t pf[4];
        const int pch = (kk * 2 + (lane >> 4)) ^ ((prow / RP) % PCH);
        ldsm_x4(pf, pb + prow * KT + pch * 8);
        const int vrow = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
        for (int nt = 0; nt < NT; nt += 2) {
          uint32_t vf[4];
          const int dch = g * (C::DW / 8) + nt + (lane >> 4);
          ldsm_x4_trans(vf, kt + vrow * D + swz_row(vrow, dch) * 8);
          mma_bf16(acc[nt], pf, vf[0], vf[1]);
          mma_bf16(acc[nt + 1], pf, vf[2], vf[3]);
        }
      }
    }
    __syncthreads();
  }
  }
  __syncthreads();
  if (nsplit > 1) {
    // leave this split's partial, then the last CTA of the token merges all of them
    __shared__ int is_last;
    const int r0 = mt * 16 + (lane >> 2);
    float* pa = a.part_acc + ((size_t)t * nsplit + split) * HL * D;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int d0 = g * C::DW + nt * 8 + (lane & 3) * 2;
      if (r0 < HL) *reinterpret_cast<float2*>(pa + (size_t)r0 * D + d0) = make_float2(acc[nt][0], acc[nt][1]);
      if (r0 + 8 < HL) *reinterpret_cast<float2*>(pa + (size_t)(r0 + 8) * D + d0) = make_float2(acc[nt][2], acc[nt][3]);
    }
    if (tid < HL) {
      float* pm = a.part_ml + (((size_t)t * nsplit + split) * HL + tid) * 2;
      pm[0] = ms[tid], pm[1] = ls[tid];
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      const int prev = atomicAdd(&a.counters[t], 1);
      is_last = prev == nsplit - 1;
      if (is_last) a.counters[t] = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // per head row: global max, rescale factors per split (kept in shared memory: alpha reused as scratch is too
    // small, so recompute per thread -- nsplit <= 32)
    float mx0 = -INFINITY, mx1 = -INFINITY;
    for (int s2 = 0; s2 < nsplit; ++s2) {
      const float* pm = a.part_ml + ((size_t)t * nsplit + s2) * HL * 2;
      if (r0 < HL) mx0 = fmaxf(mx0, __ldcg(pm + r0 * 2));
      if (r0 + 8 < HL) mx1 = fmaxf(mx1, __ldcg(pm + (r0 + 8) * 2));
    }
    float l0 = 0.f, l1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
    for (int s2 = 0; s2 < nsplit; ++s2) {
      const float* pm = a.part_ml + ((size_t)t * nsplit + s2) * HL * 2;
      const float* ps2 = a.part_acc + ((size_t)t * nsplit + s2) * HL * D;
      float w0 = 0.f, w1 = 0.f;
      if (r0 < HL) w0 = __expf(__ldcg(pm + r0 * 2) - mx0), l0 += __ldcg(pm + r0 * 2 + 1) * w0;
      if (r0 + 8 < HL) w1 = __expf(__ldcg(pm + (r0 + 8) * 2) - mx1), l1 += __ldcg(pm + (r0 + 8) * 2 + 1) * w1;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int d0 = g * C::DW + nt * 8 + (lane & 3) * 2;
        if (r0 < HL) {
          const float2 v = __ldcg(reinterpret_cast<const float2*>(ps2 + (size_t)r0 * D + d0));
          acc[nt][0] = fmaf(v.x, w0, acc[nt][0]), acc[nt][1] = fmaf(v.y, w0, acc[nt][1]);
        }
        if (r0 + 8 < HL) {
          const float2 v = __ldcg(reinterpret_cast<const float2*>(ps2 + (size_t)(r0 + 8) * D + d0));
          acc[nt][2] = fmaf(v.x, w1, acc[nt][2]), acc[nt][3] = fmaf(v.y, w1, acc[nt][3]);
        }
      }
    }
    __syncthreads();
    if ((lane & 3) == 0 && g == 0) {   // one writer per head row
      if (r0 < HL) ls[r0] = l0;
      if (r0 + 8 < HL) ls[r0 + 8] = l1;
    }
    __syncthreads();
  }
  {
    const int r0 = mt * 16 + (lane >> 2);
    const float i0 = 1.f / ls[r0], i1 = 1.f / ls[r0 + 8];
    const float fpos = a.out_rope ? (float)a.pos[t] : 0.f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int d0 = g * C::DW + nt * 8 + (lane & 3) * 2;
      __nv_bfloat162 v0 = __floats2bfloat162_rn(acc[nt][0] * i0, acc[nt][1] * i0);
      __nv_bfloat162 v1 = __floats2bfloat162_rn(acc[nt][2] * i1, acc[nt][3] * i1);
      if (a.out_rope && d0 >= D - a.rp.rotary_dim) {  // interleaved pair (d0, d0 + 1) sits in this thread
        float c, sn;
        rope_cos_sin(a.rp, fpos, (d0 - (D - a.rp.rotary_dim)) >> 1, 1, c, sn);
        const float2 f0 = __bfloat1622float2(v0), f1 = __bfloat1622float2(v1);
        v0 = __floats2bfloat162_rn(f0.x * c - f0.y * sn, f0.x * sn + f0.y * c);
        v1 = __floats2bfloat162_rn(f1.x * c - f1.y * sn, f1.x * sn + f1.y * c);
      }
      if (r0 < HL) *reinterpret_cast<__nv_bfloat162*>(a.o + ((size_t)t * HL + r0) * D + d0) = v0;
      if (r0 + 8 < HL) *reinterpret_cast<__nv_bfloat162*>(a.o + ((size_t)t * HL + r0 + 8) * D + d0) = v1;
    }
  }
}

template <int HL>
int launch_attn(const AttnArgs& a, int t, cudaStream_t st) {
  if (a.nsplit > 32) return 304;
  using C = AttnCfg<HL>;
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(sparse_attn_kernel<HL>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM) !=
        cudaSuccess)
      return 301;
    set = true;
  }
  dsv4_launch(sparse_attn_kernel<HL>, dim3(t, a.nsplit), C::NW * 32, C::SMEM, st, a);
  return (int)cudaGetLastError();
}

}  // namespace

DSV4_API int dsv4_sparse_attention(const void* q, void* o, const int* slots, const int* pos, const int* page_table,
                                   int ld_pt, const void* swa, const int* swa_map, const void* comp,
                                   const int* topk_idx, const int* topk_len, int topk_width, int mode, int ratio,
                                   const float* sink, float scale, int ps, int window, const int* num_valid, int t,
                                   int heads, int d, int out_rope, RopeParams rp, int nsplit, float* part_acc,
                                   float* part_ml, int* counters, cudaStream_t st) {
  if (t <= 0) return 0;
  if (d != D) return 300;
  if (nsplit < 1) nsplit = 1;
  if (nsplit > 1 && (!part_acc || !part_ml || !counters)) return 305;
  if (out_rope && (rp.rotary_dim <= 0 || rp.rotary_dim > 128 || rp.rotary_dim % 8)) return 303;
  AttnArgs a{(const __nv_bfloat16*)q, (__nv_bfloat16*)o, slots, pos, page_table, ld_pt, (const __nv_bfloat16*)swa,
             swa_map, (const __nv_bfloat16*)comp, topk_idx, topk_len, topk_width, mode, ratio, sink, scale, ps,
             window, num_valid, out_rope, rp, nsplit, part_acc, part_ml, counters};
  switch (heads) {
    case 8: return launch_attn<8>(a, t, st);
    case 16: return launch_attn<16>(a, t, st);
    case 32: return launch_attn<32>(a, t, st);
    case 64: return launch_attn<64>(a, t, st);
    default: return 302;
  }
}
