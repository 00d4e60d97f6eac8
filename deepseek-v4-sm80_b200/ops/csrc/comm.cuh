// In-kernel collectives over NVLink peer memory (plain P2P loads/stores through NVSwitch).
//
// Every rank owns one symmetric allocation with the same layout; `CommCtx` carries all ranks' base pointers:
//   flags  [channel][writer rank][slot]  uint32, written remotely by `writer rank`, polled locally
//   data   [channel][parity][row][col]   bf16 partial results of this rank, read remotely by every peer
// A *channel* is one call site (attention output projection, MoE combine, generic).  A call uses the channel's
// device-resident epoch E: partials go to data[E & 1], flags carry E.  Each CTA owns a set of tiles: it writes its
// partial tile locally, publishes flag[E] to every peer, waits for the same tile's flag from every peer and reduces
// the 'world' copies in rank order (so all ranks produce bit-identical sums).  A CTA only ever waits on other GPUs,
// never on a CTA of its own grid, so no co-residency of the grid is required.  Reuse of data[E & 1] two calls later is
// safe because a rank can only finish call E+1 after every peer has entered call E+1, i.e. finished call E.
// The last CTA of the grid to finish bumps the epoch, which keeps the protocol valid under CUDA-graph replay.
// All waits are bounded: on expiry the kernel records DSV4_ERR_PEER_TIMEOUT and returns without reducing.
#pragma once
#include "common.cuh"

constexpr int kMaxRanks = 8;
constexpr int kCommChannels = 3;
constexpr int kCommSlots = 8192;
constexpr int kTwoShotSlot = kCommSlots / 2;  // second-phase flags of the two-shot paths start here

struct CommCtx {
  uint8_t* peer[kMaxRanks];   // symmetric base of every rank (peer[rank] is local)
  int rank, world;
  int channel;
  int big;                    // > 0: tensors of more than `big` rows use the block-wise two-shot path (0: never)
  long long data_bytes;       // bytes of one parity buffer of one channel
  long long small_bytes;      // bytes of one result buffer of the two-shot path (0: none)
  int* epoch;                 // local [kCommChannels] device ints
  int* done;                  // local [kCommChannels] device ints
  uint8_t* mc;                // NVSwitch multicast mapping of the same allocation (null: none)
  int mm;                     // 1: reductions go through the switch (multimem.ld_reduce / multimem.st)
  int pad_;
};
static_assert(sizeof(CommCtx) == 128, "the Python side mirrors this struct field by field");

__host__ __device__ inline size_t comm_flags_bytes() { return (size_t)kCommChannels * kMaxRanks * kCommSlots * 4; }
__device__ __forceinline__ uint32_t* comm_flag(const CommCtx& c, int on_rank, int writer, int slot) {
  return reinterpret_cast<uint32_t*>(c.peer[on_rank]) + ((size_t)c.channel * kMaxRanks + writer) * kCommSlots + slot;
}
__device__ __forceinline__ __nv_bfloat16* comm_data(const CommCtx& c, int on_rank, int parity) {
  return reinterpret_cast<__nv_bfloat16*>(c.peer[on_rank] + comm_flags_bytes() +
                                          ((size_t)c.channel * 2 + parity) * (size_t)c.data_bytes);
}
// result[channel][parity] of the two-shot path: final rows, written remotely by each row's owner
__device__ __forceinline__ __nv_bfloat16* comm_result(const CommCtx& c, int on_rank, int parity) {
  return reinterpret_cast<__nv_bfloat16*>(c.peer[on_rank] + comm_flags_bytes() +
                                          (size_t)kCommChannels * 2 * (size_t)c.data_bytes +
                                          ((size_t)c.channel * 2 + parity) * (size_t)c.small_bytes);
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_peer16(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// Bulk data for a peer: a plain (weak) 16-byte store.  Unlike the volatile form it may be merged with its neighbours
// on the way to the link; the writer's system-scope fence before it raises the flag makes the data visible.
__device__ __forceinline__ void st_bulk16(void* p, const uint4& v) { *reinterpret_cast<uint4*>(p) = v; }

__device__ __forceinline__ void st_peer16(void* p, const uint4& v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// Called by ONE thread after the CTA's partial tile is written and the writers have synchronised.
__device__ __forceinline__ void comm_publish(const CommCtx& c, int slot, uint32_t epoch) {
  // one system-scope fence orders the tile before all flags; the flag stores themselves are then posted without
  // waiting for one another (a release store per peer would pay an NVLink round trip each, in series)
  __threadfence_system();
#pragma unroll
  for (int p = 0; p < kMaxRanks; ++p)
    if (p < c.world && p != c.rank) st_relaxed_sys(comm_flag(c, p, c.rank, slot), epoch);
}
// Called by ONE thread; returns false when a peer's flag did not arrive in time.  All peers' flags are polled
// together (independent relaxed loads), then one acquire fence orders the data reads after them.
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool comm_wait(const CommCtx& c, int slot, uint32_t epoch) {
  unsigned long long t0 = 0;
  for (int spin = 0;; ++spin) {
    uint32_t v[kMaxRanks];
#pragma unroll
    for (int p = 0; p < kMaxRanks; ++p)
      v[p] = (p < c.world && p != c.rank) ? ld_relaxed_sys(comm_flag(c, c.rank, p, slot)) : epoch;
    int late = -1;
#pragma unroll
    for (int p = 0; p < kMaxRanks; ++p)
      if ((int)(v[p] - epoch) < 0) late = p;
    if (late < 0) break;
    if ((spin & 63) == 63) {
      const unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > kWaitLimitNs) {
        dsv4_set_error(DSV4_ERR_PEER_TIMEOUT, late, slot);
        return false;
      }
    }
  }
  __threadfence_system();
  return true;
}
// Sum `world` bf16x8 vectors (one per rank, same offset) in rank order, fp32 accumulate, round once.
// The loads are issued back to back before the first add: a peer load takes microseconds over NVLink, and a loop that
// adds each vector before asking for the next one pays that latency `world` times.
__device__ __forceinline__ void comm_gather16(const CommCtx& c, int parity, size_t elem_offset, uint4 (&v)[kMaxRanks]) {
#pragma unroll
  for (int p = 0; p < kMaxRanks; ++p)
    if (p < c.world) v[p] = ld_peer16(comm_data(c, p, parity) + elem_offset);
}
__device__ __forceinline__ uint4 comm_sum16(const CommCtx& c, const uint4 (&v)[kMaxRanks]) {
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
  for (int p = 0; p < kMaxRanks; ++p) {
    if (p < c.world) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[p]);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(h[k]);
        acc[2 * k] += f.x;
        acc[2 * k + 1] += f.y;
      }
    }
  }
  uint4 o;
  __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int k = 0; k < 4; ++k) ho[k] = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
  return o;
}
__device__ __forceinline__ uint4 comm_reduce16(const CommCtx& c, int parity, size_t elem_offset) {
  uint4 v[kMaxRanks];
  comm_gather16(c, parity, elem_offset, v);
  return comm_sum16(c, v);
}
// Two vectors at once (16 peer loads in flight per thread).
__device__ __forceinline__ void comm_reduce16x2(const CommCtx& c, int parity, size_t off0, size_t off1, uint4& o0,
                                                uint4& o1) {
  uint4 v0[kMaxRanks], v1[kMaxRanks];
  comm_gather16(c, parity, off0, v0);
  comm_gather16(c, parity, off1, v1);
  o0 = comm_sum16(c, v0);
  o1 = comm_sum16(c, v1);
}
// Wait for ONE writer's flag (two-shot path).  Called by one thread.
__device__ __forceinline__ bool comm_wait_one(const CommCtx& c, int writer, int slot, uint32_t epoch) {
  const uint32_t* f = comm_flag(c, c.rank, writer, slot);
  unsigned long long t0 = 0;
  for (int spin = 0;; ++spin) {
    if ((int)(ld_relaxed_sys(f) - epoch) >= 0) break;
    if ((spin & 63) == 63) {
      const unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > kWaitLimitNs) {
        dsv4_set_error(DSV4_ERR_PEER_TIMEOUT, writer, slot);
        return false;
      }
    }
  }
  __threadfence_system();
  return true;
}

// ---------------------------------------------------------------- in-switch reduction (NVLS)
// The multicast mapping `c.mc` addresses the same offset of the symmetric allocation on EVERY rank at once:
//   multimem.st        writes a value to all ranks' copies (one instruction instead of world-1 peer stores),
//   multimem.ld_reduce makes the switch load all ranks' copies, add them and return the sum.
// Flags keep the layout and the epoch protocol of the peer-to-peer paths, so both kinds of call can share a channel.
__device__ __forceinline__ uint32_t* comm_mc_flag(const CommCtx& c, int writer, int slot) {
  return reinterpret_cast<uint32_t*>(c.mc) + ((size_t)c.channel * kMaxRanks + writer) * kCommSlots + slot;
}
__device__ __forceinline__ __nv_bfloat16* comm_mc_data(const CommCtx& c, int parity) {
  return reinterpret_cast<__nv_bfloat16*>(c.mc + comm_flags_bytes() +
                                          ((size_t)c.channel * 2 + parity) * (size_t)c.data_bytes);
}
__device__ __forceinline__ void mm_st_u32(uint32_t* p, uint32_t v) {
  asm volatile("multimem.st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void mm_st16(void* p, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}
// Sum of the 8 bf16 values at this offset over all ranks, accumulated in fp32 inside the switch.
__device__ __forceinline__ uint4 mm_ld_reduce16(const void* p) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ bool comm_use_multimem(const CommCtx& c, int rows, int cols) {
  return c.mm && c.mc != nullptr && c.world > 1 && rows <= kTwoShotSlot && rows <= (int)gridDim.x && cols % 8 == 0;
}
// One-shot all-reduce of ONE row by ONE CTA through the switch (all threads call it; the CTA's partial row already
// sits in comm_data(rank, parity) and the CTA has synchronised).  One multicast store raises this rank's flag on every
// rank; once the world-1 other flags arrived, every rank asks the switch for the sum of the row.  One NVLink round
// trip for the flags and one for the data, against two each on the two-shot path.  Every rank issues the same
// ld_reduce, and the switch adds the ranks' copies in a fixed order, so all ranks receive the same bits (the
// communicator checks this once at start-up and otherwise stays on the peer-to-peer paths).
template <class Emit>
__device__ __forceinline__ void comm_row_multimem(const CommCtx& c, uint32_t epoch, int row, int cols, int* sh_ok,
                                                  Emit emit) {
  const int parity = epoch & 1;
  if (threadIdx.x == 0) {
    __threadfence_system();
    mm_st_u32(comm_mc_flag(c, c.rank, row), epoch);
    *sh_ok = comm_wait(c, row, epoch) ? 1 : 0;
  }
  __syncthreads();
  if (!*sh_ok) return;
  const __nv_bfloat16* src = comm_mc_data(c, parity) + (size_t)row * cols;
  for (int i = threadIdx.x * 8; i < cols; i += blockDim.x * 16) {
    const int i1 = i + blockDim.x * 8;
    const uint4 v0 = mm_ld_reduce16(src + i);
    if (i1 < cols) {
      const uint4 v1 = mm_ld_reduce16(src + i1);
      emit(i1, v1);
    }
    emit(i, v0);
  }
}

// Two-shot all-reduce of ONE row by ONE CTA (all threads call it; the CTA's partial row already sits in
// comm_data(rank, parity) and the CTA has synchronised).  Row r is owned by rank r % world: the owner waits for the
// 7 partials, sums them in rank order, writes the result row into every rank's result buffer and raises a second
// flag; the other ranks only tell the owner that their partial is ready and wait for that second flag.  Per rank
// this moves 2 * (world-1)/world of the tensor over NVLink instead of (world-1) times the tensor, and a non-owner
// sends one flag instead of world-1.  emit(col, v) receives 8 reduced bf16 values of the row.
template <class Emit>
__device__ __forceinline__ void comm_row_two_shot(const CommCtx& c, uint32_t epoch, int row, int cols, int* sh_ok,
                                                  Emit emit) {
  const int parity = epoch & 1, owner = row % c.world;
  if (threadIdx.x == 0) {
    __threadfence_system();
    int ok;
    if (owner != c.rank) {
      st_relaxed_sys(comm_flag(c, owner, c.rank, row), epoch);
      ok = comm_wait_one(c, owner, kTwoShotSlot + row, epoch) ? 1 : 0;
    } else {
      ok = comm_wait(c, row, epoch) ? 1 : 0;
    }
    *sh_ok = ok;
  }
  __syncthreads();
  if (!*sh_ok) return;
  const size_t off = (size_t)row * cols;
  if (owner == c.rank) {
    for (int i = threadIdx.x * 8; i < cols; i += blockDim.x * 16) {
      const int i1 = i + blockDim.x * 8;
      uint4 v0, v1 = make_uint4(0, 0, 0, 0);
      if (i1 < cols)
        comm_reduce16x2(c, parity, off + i, off + i1, v0, v1);
      else
        v0 = comm_reduce16(c, parity, off + i);
#pragma unroll
      for (int p = 0; p < kMaxRanks; ++p) {
        if (p < c.world && p != c.rank) {
          __nv_bfloat16* dst = comm_result(c, p, parity) + off;
          st_peer16(dst + i, v0);
          if (i1 < cols) st_peer16(dst + i1, v1);
        }
      }
      emit(i, v0);
      if (i1 < cols) emit(i1, v1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
#pragma unroll
      for (int p = 0; p < kMaxRanks; ++p)
        if (p < c.world && p != c.rank) st_relaxed_sys(comm_flag(c, p, c.rank, kTwoShotSlot + row), epoch);
    }
  } else {
    const __nv_bfloat16* src = comm_result(c, c.rank, parity) + off;
    for (int i = threadIdx.x * 8; i < cols; i += blockDim.x * 8) emit(i, ld_peer16(src + i));
  }
}
__device__ __forceinline__ bool comm_use_two_shot(const CommCtx& c, int rows, int cols) {
  return c.world >= 4 && c.small_bytes > 0 && rows <= 256 && rows <= (int)gridDim.x &&
         (long long)rows * cols * 2 <= c.small_bytes;
}

// Two-shot all-reduce of a LARGE tensor (prefill: thousands of rows) by blocks of rows.  All CTAs of the grid call it
// with all threads.  Block b = rows [b * R, (b + 1) * R) belongs to CTA b % grid in its pass b / grid, on every rank
// alike, and is owned by rank (b % grid + b / grid) % world, which spreads each CTA's owned blocks over the ranks.
//   phase A, per block: deposit(r0, r1) puts this rank's partial rows into its parity buffer (a no-op when an earlier
//     kernel did that); a non-owner then raises flag[b] at the owner; the owner waits for the world-1 flags, sums the
//     partials in rank order, stores the result rows IN PLACE into every peer's parity buffer (only the owner ever
//     reads a block's partials, and each 16-byte piece is read before it is overwritten), emits them locally and
//     raises flag[half + b] at every peer.
//   phase B, per block not owned: wait for the owner's second flag, emit the rows from the own parity buffer.
// Phase A never waits for a phase B, and a block's partials only need pass k of the same CTA index on the peers, so
// the exchange makes progress whenever the grid is co-resident (the launchers size it so); every wait is bounded.
// Per rank this moves 2 * (world-1)/world of the tensor over NVLink; the one-shot form moves (world-1) times it.
// emit(row, col, v) receives 8 reduced bf16 values.
// Rows per block: every block costs two flag exchanges, so large tensors use larger blocks (about two passes per CTA
// at 8 192 rows) and small ones use 8-, 4- or 2-row blocks so that a hundred or more CTAs have work.
__host__ __device__ __forceinline__ int comm_big_block_rows(int rows) {
  int r = rows > 4096 ? 32 : rows > 2048 ? 16 : rows > 512 ? 8 : rows > 256 ? 4 : 2;
  while ((rows + r - 1) / r > kTwoShotSlot) r *= 2;
  return r;
}
inline bool comm_host_use_big(const CommCtx& c, int rows) { return c.world > 1 && c.big > 0 && rows > c.big; }
// With c.mm set, the owner's reduction is one multimem.ld_reduce per 16 bytes (the switch adds the ranks' partials)
// and its result goes to all ranks with one multimem.st; the second flag is one multicast store as well.  Per rank
// that is (world-1)/world of the tensor in each NVLink direction, half of what the peer-to-peer form moves.
template <class Deposit, class Emit>
__device__ __forceinline__ void comm_big_two_shot(const CommCtx& c, uint32_t epoch, int rows, int cols, int* sh_ok,
                                                  Deposit deposit, Emit emit) {
  const bool use_mm = c.mm && c.mc != nullptr;
  const int parity = epoch & 1, G = gridDim.x, R = comm_big_block_rows(rows), nblk = (rows + R - 1) / R;
  __nv_bfloat16* mine = comm_data(c, c.rank, parity);
  for (int b = blockIdx.x, k = 0; b < nblk; b += G, ++k) {
    const int r0 = b * R, r1 = min(rows, r0 + R), owner = (int)((blockIdx.x + k) % c.world);
    deposit(r0, r1);
    __syncthreads();
    if (threadIdx.x == 0) {
      int ok = 1;
      if (owner != c.rank) {
        __threadfence_system();
        st_relaxed_sys(comm_flag(c, owner, c.rank, b), epoch);
      } else {
        ok = comm_wait(c, b, epoch) ? 1 : 0;
      }
      *sh_ok = ok;
    }
    __syncthreads();
    const int ok = *sh_ok;
    if (owner == c.rank && ok && use_mm) {
      // the block's rows are contiguous: eight independent switch reductions per thread and trip (a reduction is a
      // round trip through the switch, so the bytes in flight per SM decide the rate)
      constexpr int U = 8;
      const int c8 = cols / 8, n8 = (r1 - r0) * c8;
      __nv_bfloat16* mcb = comm_mc_data(c, parity) + (size_t)r0 * cols;
      for (int i = threadIdx.x; i < n8; i += blockDim.x * U) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int j = i + u * (int)blockDim.x;
          if (j < n8) v[u] = mm_ld_reduce16(mcb + (size_t)j * 8);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int j = i + u * (int)blockDim.x;
          if (j < n8) {
            mm_st16(mcb + (size_t)j * 8, v[u]);
            emit(r0 + j / c8, (j % c8) * 8, v[u]);
          }
        }
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        __threadfence_system();
        mm_st_u32(comm_mc_flag(c, c.rank, kTwoShotSlot + b), epoch);
      }
    } else if (owner == c.rank && ok) {
      for (int r = r0; r < r1; ++r) {
        const size_t off = (size_t)r * cols;
        for (int i = threadIdx.x * 8; i < cols; i += blockDim.x * 16) {
          const int i1 = i + blockDim.x * 8;
          uint4 v0, v1 = make_uint4(0, 0, 0, 0);
          if (i1 < cols)
            comm_reduce16x2(c, parity, off + i, off + i1, v0, v1);
          else
            v0 = comm_reduce16(c, parity, off + i);
#pragma unroll
          for (int p = 0; p < kMaxRanks; ++p) {
            if (p < c.world && p != c.rank) {
              __nv_bfloat16* dst = comm_data(c, p, parity) + off;
              st_peer16(dst + i, v0);
              if (i1 < cols) st_peer16(dst + i1, v1);
            }
          }
          emit(r, i, v0);
          if (i1 < cols) emit(r, i1, v1);
        }
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        __threadfence_system();
#pragma unroll
        for (int p = 0; p < kMaxRanks; ++p)
          if (p < c.world && p != c.rank) st_relaxed_sys(comm_flag(c, p, c.rank, kTwoShotSlot + b), epoch);
      }
    }
    __syncthreads();  // *sh_ok is rewritten by the next pass
    if (!ok) return;  // uniform over the CTA; the status word already holds the timeout
  }
  for (int b = blockIdx.x, k = 0; b < nblk; b += G, ++k) {
    const int r0 = b * R, r1 = min(rows, r0 + R), owner = (int)((blockIdx.x + k) % c.world);
    if (owner == c.rank) continue;
    if (threadIdx.x == 0) *sh_ok = comm_wait_one(c, owner, kTwoShotSlot + b, epoch) ? 1 : 0;
    __syncthreads();
    const int ok = *sh_ok;
    if (ok) {
      // the block's rows are contiguous: four independent 16-byte loads per thread and trip
      const int c8 = cols / 8, n8 = (r1 - r0) * c8;
      const uint4* src = reinterpret_cast<const uint4*>(mine + (size_t)r0 * cols);
      for (int i = threadIdx.x; i < n8; i += blockDim.x * 4) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int j = i + u * (int)blockDim.x;
          if (j < n8) v[u] = ld_peer16(src + j);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int j = i + u * (int)blockDim.x;
          if (j < n8) emit(r0 + j / c8, (j % c8) * 8, v[u]);
        }
      }
    }
    __syncthreads();
    if (!ok) return;
  }
}
// Grid of a kernel on the block-wise path: one CTA of 256 threads per SM at most, so that all of them are co-resident.
inline int comm_big_grid(int rows) {
  const int r = comm_big_block_rows(rows);
  const int nblk = (rows + r - 1) / r;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return nblk < sms ? nblk : sms;
}

// ---------------------------------------------------------------- row-sharded (sequence-parallel) exchange
// Between the two collectives of a block the layer can keep its activations sharded by rows: rank r owns the rows
// [r * rows_per_rank, (r + 1) * rows_per_rank) (a multiple of 128, so that a 128-row GEMM tile has one owner).
//   reduce-scatter: a producer (projection GEMM epilogue, MoE combine) stores each partial row straight into the
//     OWNER's buffer rs[src rank][local row][col] over NVLink and, once a 128-row block is complete, raises
//     flag[RS][src][local block] at the owner; the owner adds the `world` partials in rank order (sp.cu).
//   all-gather: the owner pushes its finished rows (bf16, e4m3 and scales) into every rank's gathered buffer and
//     raises flag[AG][owner][global block] everywhere; the consuming GEMM's TMA producer waits for the flag of its
//     row block before it loads the block's A tiles (gemm_tcgen05.cu), weights streaming in the meantime.
// These calls are issued eagerly (prefill), so the host numbers them: `seq` is a counter that all ranks advance
// alike, flags carry it, and a waiter accepts any value >= its own.  All waits are bounded.
constexpr int kSpSlots = 256;
enum { kSpAG = 0, kSpRS = 1 };
struct SpCtx {
  uint8_t* peer[kMaxRanks];
  uint8_t* mc;            // multicast mapping (null: plain peer stores)
  int rank, world;
  int rows_per_rank;      // multiple of 128
  int hidden;
  long long flags_off;    // uint32 [2 kinds][kMaxRanks writers][kSpSlots]
  long long ag_off;       // gathered rows of this channel: bf16 [tpad, hidden] | u8 [tpad, hidden] | f32 [tpad, hidden/128]
  long long rs_off;       // partial rows of this channel: bf16 [world][rows_per_rank][hidden]
  unsigned int seq;
  int use_mc;             // 1: pushes and flags go through multimem.st
};
static_assert(sizeof(SpCtx) == 120, "the Python side mirrors this struct field by field");
__device__ __forceinline__ uint32_t* sp_flag(const SpCtx& c, int on_rank, int kind, int writer, int slot) {
  return reinterpret_cast<uint32_t*>(c.peer[on_rank] + c.flags_off) + ((size_t)kind * kMaxRanks + writer) * kSpSlots +
         slot;
}
__device__ __forceinline__ uint32_t* sp_mc_flag(const SpCtx& c, int kind, int writer, int slot) {
  return reinterpret_cast<uint32_t*>(c.mc + c.flags_off) + ((size_t)kind * kMaxRanks + writer) * kSpSlots + slot;
}
// Bounded wait on ONE local flag word (any value >= seq passes).  Called by one thread.
__device__ __forceinline__ bool sp_wait_flag(const uint32_t* f, uint32_t seq, int who, int slot) {
  unsigned long long t0 = 0;
  for (int spin = 0;; ++spin) {
    if ((int)(ld_relaxed_sys(f) - seq) >= 0) break;
    if ((spin & 63) == 63) {
      const unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > kWaitLimitNs) {
        dsv4_set_error(DSV4_ERR_PEER_TIMEOUT, who, slot);
        return false;
      }
    }
  }
  __threadfence_system();
  return true;
}

// Last CTA of the grid advances the channel epoch (call once per CTA, by one thread, at the very end).
__device__ __forceinline__ void comm_finish(const CommCtx& c, int total_ctas) {
  __threadfence();
  if (atomicAdd(&c.done[c.channel], 1) == total_ctas - 1) {
    c.done[c.channel] = 0;
    __threadfence();
    atomicAdd(&c.epoch[c.channel], 1);
  }
}
__device__ __forceinline__ uint32_t comm_epoch(const CommCtx& c) {
  return (uint32_t)(*reinterpret_cast<volatile int*>(&c.epoch[c.channel])) + 1u;
}
