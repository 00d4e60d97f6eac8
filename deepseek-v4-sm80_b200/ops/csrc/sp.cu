// Row-sharded (sequence-parallel) layer exchange: the all-gather push of a rank's finished rows and the owner-side
// reduction of the partial rows a reduce-scatter delivered.  The producers of the reduce-scatter live in
// gemm_tcgen05.cu (projection epilogue) and moe.cu (expert combine), the consumer of the all-gather is the gated
// A-tile load of gemm_tcgen05.cu.  Layout and protocol: comm.cuh.  The reference keeps activations replicated and
// all-reduces them (python/minisgl/models/deepseek_v4.py:488-492, :916-922, :1475-1491).
#include "comm.cuh"
#include "hc_post.cuh"

namespace {

__device__ __forceinline__ void sp_store16_all(const SpCtx& c, size_t off, const uint4& v) {
  if (c.use_mc) {
    mm_st16(c.mc + off, v);   // lands in every rank's copy, this rank's included
  } else {
#pragma unroll
    for (int p = 0; p < kMaxRanks; ++p)
      if (p < c.world && p != c.rank) st_bulk16(c.peer[p] + off, v);
  }
}

// One CTA pushes a slab of this rank's rows of the gathered buffer (already written locally by the producing kernel)
// to all peers; the last CTA of a 128-row block raises the block's flag on every rank.
// grid = (rows_per_rank / 128, kParts).
constexpr int kParts = 8;
__global__ void __launch_bounds__(256) sp_ag_push_kernel(const SpCtx c, int tpad, int* __restrict__ counters) {
  pdl_entry();
  const int blk = blockIdx.x, part = blockIdx.y;
  const int h = c.hidden;
  const int row0 = c.rank * c.rows_per_rank + blk * 128 + part * (128 / kParts);
  const size_t y_off = c.ag_off, q_off = c.ag_off + (size_t)tpad * h * 2, s_off = q_off + (size_t)tpad * h;
  const uint8_t* mine = c.peer[c.rank];
  for (int r = 0; r < 128 / kParts; ++r) {
    const int row = row0 + r;
    const size_t yo = y_off + (size_t)row * h * 2, qo = q_off + (size_t)row * h, so = s_off + (size_t)row * (h / 128) * 4;
    const int ny = h * 2 / 16, nq = h / 16, ns = (h / 128) * 4 / 16;
    for (int i = threadIdx.x; i < ny + nq + ns; i += blockDim.x) {
      const size_t off = i < ny ? yo + (size_t)i * 16 : i < ny + nq ? qo + (size_t)(i - ny) * 16 : so + (size_t)(i - ny - nq) * 16;
      sp_store16_all(c, off, *reinterpret_cast<const uint4*>(mine + off));
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(&counters[blk], 1) == kParts - 1) {
      counters[blk] = 0;
      __threadfence_system();
      const int slot = c.rank * (c.rows_per_rank / 128) + blk;
      if (c.use_mc) {
        mm_st_u32(sp_mc_flag(c, kSpAG, c.rank, slot), c.seq);
      } else {
#pragma unroll
        for (int p = 0; p < kMaxRanks; ++p)
          if (p < c.world && p != c.rank) st_relaxed_sys(sp_flag(c, p, kSpAG, c.rank, slot), c.seq);
      }
    }
  }
}

// Owner side of the reduce-scatter: CTA r adds the `world` partials of local row r in rank order (all of them sit in
// this rank's own buffer) and writes the row, or -- with the hyper-connection arguments -- the new residual streams.
// mc_mode: the producers left their partials in their own buffers ([T, cols] at the same offset on every rank) and the
// switch adds them (multimem.ld_reduce on the multicast mapping), instead of the ranks' partials sitting here.
__global__ void __launch_bounds__(256) sp_rs_reduce_kernel(const SpCtx c, int cols, __nv_bfloat16* __restrict__ out,
                                                           const HcPostArgs hc, int mc_mode) {
  pdl_entry();
  __shared__ int ok;
  const int row = blockIdx.x, blk = row >> 7;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < c.world) {
    // thread p waits for writer p (this rank's own producer raises the local flag like any other writer)
    if (!sp_wait_flag(sp_flag(c, c.rank, kSpRS, threadIdx.x, blk), c.seq, threadIdx.x, blk)) atomicExch(&ok, 0);
  }
  __syncthreads();
  if (!ok) return;
  if (mc_mode) {
    const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(c.mc + c.rs_off) +
                               ((size_t)c.rank * c.rows_per_rank + row) * cols;
    for (int i = threadIdx.x * 8; i < cols; i += blockDim.x * 16) {
      const int i1 = i + blockDim.x * 8;
      const uint4 v0 = mm_ld_reduce16(src + i);
      uint4 v1 = make_uint4(0, 0, 0, 0);
      if (i1 < cols) v1 = mm_ld_reduce16(src + i1);
      if (hc.res) {
        hc_post_store8(v0, hc, row, cols, i);
        if (i1 < cols) hc_post_store8(v1, hc, row, cols, i1);
      } else {
        *reinterpret_cast<uint4*>(out + (size_t)row * cols + i) = v0;
        if (i1 < cols) *reinterpret_cast<uint4*>(out + (size_t)row * cols + i1) = v1;
      }
    }
    return;
  }
  const __nv_bfloat16* base = reinterpret_cast<const __nv_bfloat16*>(c.peer[c.rank] + c.rs_off);
  for (int i = threadIdx.x * 8; i < cols; i += blockDim.x * 8) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    uint4 v[kMaxRanks];
#pragma unroll
    for (int p = 0; p < kMaxRanks; ++p)
      if (p < c.world) v[p] = ld_peer16(base + ((size_t)p * c.rows_per_rank + row) * cols + i);
#pragma unroll
    for (int p = 0; p < kMaxRanks; ++p) {
      if (p < c.world) {
        const __nv_bfloat162* hp = reinterpret_cast<const __nv_bfloat162*>(&v[p]);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = __bfloat1622float2(hp[k]);
          acc[2 * k] += f.x, acc[2 * k + 1] += f.y;
        }
      }
    }
    uint4 o;
    __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int k = 0; k < 4; ++k) ho[k] = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
    if (hc.res)
      hc_post_store8(o, hc, row, cols, i);
    else
      *reinterpret_cast<uint4*>(out + (size_t)row * cols + i) = o;
  }
}

}  // namespace

DSV4_API int dsv4_sp_ctx_size() { return (int)sizeof(SpCtx); }
DSV4_API int dsv4_sp_slots() { return kSpSlots; }

// Pushes this rank's rows [rank * rows_per_rank, +rows_per_rank) of the gathered buffer (bf16 rows, e4m3 rows and
// scales, written locally by the kernels before this one) to every peer and raises the per-block flags.
// counters: >= rows_per_rank / 128 zeroed ints.
DSV4_API int dsv4_sp_ag_push(const SpCtx* c, int tpad, int* counters, cudaStream_t st) {
  if (c->world <= 1) return 0;
  if (c->rows_per_rank % 128 || c->hidden % 512 || tpad != c->rows_per_rank * c->world) return 520;
  if (tpad / 128 > kSpSlots) return 521;
  dsv4_launch(sp_ag_push_kernel, dim3(c->rows_per_rank / 128, kParts), 256, 0, st, *c, tpad, counters);
  return (int)cudaGetLastError();
}

// Reduces the partial rows delivered to this rank: rows = valid local rows.  out bf16 [rows, cols], or with
// res / post / comb / xout the hyper-connection post mix of the reduced rows ([rows, 4, cols]).
DSV4_API int dsv4_sp_rs_reduce(const SpCtx* c, int rows, int cols, void* out, const void* res, const float* post,
                               const float* comb, void* xout, int mc_mode, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (cols % 8 || rows > c->rows_per_rank) return 522;
  if (xout && (!res || !post || !comb)) return 523;
  HcPostArgs hc{xout ? (const __nv_bfloat16*)res : nullptr, post, comb, (__nv_bfloat16*)xout};
  if (mc_mode && !(c->use_mc && c->mc)) return 524;
  dsv4_launch(sp_rs_reduce_kernel, rows, 256, 0, st, *c, cols, (__nv_bfloat16*)out, hc, mc_mode);
  return (int)cudaGetLastError();
}
