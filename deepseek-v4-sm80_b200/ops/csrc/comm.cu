// Stand-alone in-kernel all-reduce over NVLink peer memory (bf16 [rows, cols], sum), using the protocol in comm.cuh.
// It is the unfused form of the two fused call sites (projection GEMM epilogue in gemm_tcgen05.cu, MoE combine in
// moe.cu), used for the embedding-free generic reductions, for tests and as the microbenchmark baseline against
// NCCL.  Each CTA owns rows b, b + grid, ...: copy to the symmetric buffer, publish, wait, reduce in rank order.
#include "comm.cuh"
#include "hc_post.cuh"

namespace {

// BIG: the block-wise two-shot path for tensors of more than comm.big rows (own instantiation: the row-wise paths of a
// decode step keep their register allocation).
template <bool BIG>
__global__ void __launch_bounds__(256) allreduce_kernel(const __nv_bfloat16* __restrict__ x,
                                                        __nv_bfloat16* __restrict__ out, int rows, int cols,
                                                        const HcPostArgs hc, const CommCtx comm) {
  pdl_entry();
  __shared__ int ok;
  const uint32_t epoch = comm_epoch(comm);
  const int parity = epoch & 1;
  __nv_bfloat16* mine = comm_data(comm, comm.rank, parity);
  const int c8 = cols / 8;
  // x == null: the producer (a GEMM in deposit mode) already wrote this rank's partial into `mine`
  auto deposit = [&](int r0, int r1) {  // rows [r0, r1) are contiguous; four loads in flight per thread
    if (!x) return;
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)r0 * cols);
    uint4* dst = reinterpret_cast<uint4*>(mine + (size_t)r0 * cols);
    const int n8 = (r1 - r0) * c8;
    for (int i = threadIdx.x; i < n8; i += blockDim.x * 4) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int j = i + u * (int)blockDim.x;
        if (j < n8) v[u] = src[j];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int j = i + u * (int)blockDim.x;
        if (j < n8) dst[j] = v[u];
      }
    }
  };
  auto emit = [&](int r, int col, const uint4& v) {
    if (hc.res)
      hc_post_store8(v, hc, r, cols, col);
    else
      *reinterpret_cast<uint4*>(out + (size_t)r * cols + col) = v;
  };
  if constexpr (BIG) {
    comm_big_two_shot(comm, epoch, rows, cols, &ok, deposit, emit);
  } else {
    for (int r = blockIdx.x; r < rows; r += gridDim.x) deposit(r, r + 1);
    __syncthreads();
    if (comm_use_multimem(comm, rows, cols)) {
      const int r = blockIdx.x;
      if (r < rows) comm_row_multimem(comm, epoch, r, cols, &ok, [&](int col, const uint4& v) { emit(r, col, v); });
    } else if (comm_use_two_shot(comm, rows, cols)) {
      const int r = blockIdx.x;
      if (r < rows) comm_row_two_shot(comm, epoch, r, cols, &ok, [&](int col, const uint4& v) { emit(r, col, v); });
    } else {
      if (threadIdx.x == 0) {
        comm_publish(comm, blockIdx.x, epoch);
        ok = comm_wait(comm, blockIdx.x, epoch) ? 1 : 0;
      }
      __syncthreads();
      if (ok) {
        for (int r = blockIdx.x; r < rows; r += gridDim.x) {
          for (int i = threadIdx.x; i < c8; i += 2 * blockDim.x) {
            const int i1 = i + blockDim.x;
            uint4 o0, o1;
            if (i1 < c8) {
              comm_reduce16x2(comm, parity, (size_t)r * cols + i * 8, (size_t)r * cols + i1 * 8, o0, o1);
              emit(r, i1 * 8, o1);
            } else {
              o0 = comm_reduce16(comm, parity, (size_t)r * cols + i * 8);
            }
            emit(r, i * 8, o0);
          }
        }
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) comm_finish(comm, gridDim.x);
}

// Greedy sampling fused behind the vocabulary-parallel LM head.  Every rank holds the logits of its own vocabulary
// shard; instead of all-gathering [rows, vocab] fp32 and taking the argmax of the whole row, each rank takes the
// argmax of its shard (one CTA per row), pushes the (value, global index) pair -- 8 bytes -- into every peer's symmetric
// buffer, and picks the best of the `world` candidates (largest value, lowest index on ties: the same rule as the
// single-rank argmax, so all ranks agree).  The winning token is written to out[row] and to token_feedback[slots[row]],
// from where the next step's embedding gathers it.  world == 1: no exchange.
__global__ void __launch_bounds__(1024) greedy_tokens_kernel(const float* __restrict__ logits, int ld, int v_local,
                                                             int v_base, const int* __restrict__ slots,
                                                             const int* __restrict__ num_valid,
                                                             int* __restrict__ token_feedback, int* __restrict__ out,
                                                             int rows, const CommCtx comm) {
  pdl_entry();
  __shared__ float sv[32];
  __shared__ int si[32];
  const int row = blockIdx.x;
  const float* lr = logits + (size_t)row * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < v_local; i += blockDim.x) {
    const float x = lr[i];
    if (x > best || (x == best && i < bi)) best = x, bi = i;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ob > best || (ob == best && oi < bi)) best = ob, bi = oi;
  }
  if ((threadIdx.x & 31) == 0) sv[threadIdx.x >> 5] = best, si[threadIdx.x >> 5] = bi;
  __syncthreads();
  if (threadIdx.x >= 32) return;
  best = threadIdx.x < (blockDim.x >> 5) ? sv[threadIdx.x] : -INFINITY;
  bi = threadIdx.x < (blockDim.x >> 5) ? si[threadIdx.x] : 0x7fffffff;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ob > best || (ob == best && oi < bi)) best = ob, bi = oi;
  }
  if (threadIdx.x != 0) return;
  int tok = bi == 0x7fffffff ? 0 : bi + v_base;
  if (comm.world > 1) {
    const uint32_t epoch = comm_epoch(comm);
    const int parity = epoch & 1;
    // candidate table of this call on every rank: [writer rank][row] of (value bits, token)
    const uint2 mine = make_uint2(__float_as_uint(best), (uint32_t)tok);
    for (int p = 0; p < comm.world; ++p) {
      uint2* tab = reinterpret_cast<uint2*>(comm_data(comm, p, parity));
      asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(tab + (size_t)comm.rank * rows + row),
                   "r"(mine.x), "r"(mine.y)
                   : "memory");
    }
    comm_publish(comm, row, epoch);
    if (comm_wait(comm, row, epoch)) {
      const uint2* tab = reinterpret_cast<const uint2*>(comm_data(comm, comm.rank, parity));
      float bv = -INFINITY;
      int bt = 0x7fffffff;
      for (int p = 0; p < comm.world; ++p) {
        uint2 c;
        asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];"
                     : "=r"(c.x), "=r"(c.y)
                     : "l"(tab + (size_t)p * rows + row)
                     : "memory");
        const float v = __uint_as_float(c.x);
        if (v > bv || (v == bv && (int)c.y < bt)) bv = v, bt = (int)c.y;
      }
      tok = bt == 0x7fffffff ? 0 : bt;
    }
    comm_finish(comm, gridDim.x);
  }
  out[row] = tok;
  if (!num_valid || row < *num_valid) token_feedback[slots[row]] = tok;
}

// A wait that nothing satisfies: used by the failure-detection test to show that a missing peer ends in an error
// status (DSV4_ERR_PEER_TIMEOUT) within `limit_ns`, with the context still usable.  It polls a LOCAL flag.
__global__ void wait_flag_kernel(const uint32_t* flag, uint32_t want, unsigned long long limit_ns, int* result) {
  pdl_entry();
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
    if (ld_acquire_sys(flag) == want) {
      *result = 1;
      return;
    }
    if (globaltimer_ns() - t0 > limit_ns) {
      dsv4_set_error(DSV4_ERR_PEER_TIMEOUT, -1, 0);
      *result = 0;
      return;
    }
  }
}

}  // namespace

DSV4_API int dsv4_comm_layout(long long* flags_bytes, int* channels, int* slots, int* max_ranks) {
  *flags_bytes = (long long)comm_flags_bytes();
  *channels = kCommChannels;
  *slots = kCommSlots;
  *max_ranks = kMaxRanks;
  return 0;
}

DSV4_API int dsv4_comm_ctx_size() { return (int)sizeof(CommCtx); }

// x may be null when this rank's partial is already in the channel's symmetric buffer (a GEMM launched in deposit
// mode on the same channel wrote it).  res / post / comb / xout (all null or all given): the hyper-connection post
// mix is applied to the reduced rows and xout [rows, 4, cols] is written instead of out.
DSV4_API int dsv4_allreduce(const void* x, void* out, int rows, int cols, const void* res, const float* post,
                            const float* comb, void* xout, const CommCtx* comm, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (cols % 8) return 500;
  if ((long long)rows * cols * 2 > comm->data_bytes) return 501;
  if (xout && (!res || !post || !comb)) return 502;
  HcPostArgs hc{xout ? (const __nv_bfloat16*)res : nullptr, post, comb, (__nv_bfloat16*)xout};
  if (comm_host_use_big(*comm, rows))
    dsv4_launch(allreduce_kernel<true>, comm_big_grid(rows), 256, 0, st, (const __nv_bfloat16*)x, (__nv_bfloat16*)out,
                rows, cols, hc, *comm);
  else
    dsv4_launch(allreduce_kernel<false>, rows < 1024 ? rows : 1024, 256, 0, st, (const __nv_bfloat16*)x,
                (__nv_bfloat16*)out, rows, cols, hc, *comm);
  return (int)cudaGetLastError();
}

// logits fp32 [rows, ld >= v_local]: this rank's vocabulary shard, whose first column is token v_base.
// comm == null or world == 1: plain argmax.  Writes out[rows] (int32) and token_feedback[slots[row]] for valid rows.
DSV4_API int dsv4_greedy_tokens(const float* logits, int ld, int v_local, int v_base, const int* slots,
                                const int* num_valid, int* token_feedback, int* out, int rows, const CommCtx* comm,
                                cudaStream_t st) {
  if (rows <= 0) return 0;
  CommCtx c{};
  c.world = 1;
  if (comm) c = *comm;
  if (c.world > 1 && (rows > kCommSlots || (long long)rows * c.world * 8 > c.data_bytes)) return 503;
  dsv4_launch(greedy_tokens_kernel, rows, 1024, 0, st, logits, ld, v_local, v_base, slots, num_valid, token_feedback, out,
              rows, c);
  return (int)cudaGetLastError();
}

DSV4_API int dsv4_wait_flag(const void* flag, unsigned want, long long limit_ns, int* result, cudaStream_t st) {
  dsv4_launch(wait_flag_kernel, 1, 1, 0, st, (const uint32_t*)flag, want, (unsigned long long)limit_ns, result);
  return (int)cudaGetLastError();
}
