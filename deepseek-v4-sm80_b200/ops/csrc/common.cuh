// Shared device/host helpers for the sm_100a kernels of this library.
//
// Everything here is plain CUDA C++ plus inline PTX for the Blackwell-only
// instructions (mbarrier, TMA bulk-tensor copies, tcgen05 MMA / TMEM).  The
// kernels are exported as `extern "C"` launchers taking raw device pointers
// and a stream, and are loaded from Python through ctypes.
//
// Every wait in this file is bounded: a wait that does not complete within
// its limit (about two seconds) records where it gave up in `g_dsv4_status` and returns
// false, and the calling kernel then unwinds (frees TMEM, returns) instead of
// spinning forever.  The host reads the status word with dsv4_read_status().
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define DSV4_API extern "C" __attribute__((visibility("default")))

// status word layout: [0] first error code (0 = ok), [1] detail a, [2] detail b, [3] count
enum Dsv4Status : int {
  DSV4_OK = 0,
  DSV4_ERR_WAIT_TIMEOUT = 1,   // a bounded mbarrier / flag wait ran out
  DSV4_ERR_BAD_INDEX = 2,      // a gathered index was out of range (checked builds)
  DSV4_ERR_PEER_TIMEOUT = 3,   // a wait on a peer GPU's flag ran out
};

extern __device__ int g_dsv4_status[8];

__device__ __forceinline__ void dsv4_set_error(int code, int a, int b) {
  if (atomicCAS(&g_dsv4_status[0], 0, code) == 0) {
    g_dsv4_status[1] = a;
    g_dsv4_status[2] = b;
  }
  atomicAdd(&g_dsv4_status[3], 1);
}

// Limit of a wait on another GPU's flag, in nanoseconds: 2 s unless dsv4_set_peer_wait_ms() changed it.
extern __device__ unsigned long long g_dsv4_peer_wait_ns;
#define kWaitLimitNs g_dsv4_peer_wait_ns
constexpr long long kWaitLimitCycles = 4000000000ll;         // 2-3 s of SM clock (waits inside one CTA)

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (and records an error) if the phase did not
// complete within the limit or if another thread of the CTA already gave up.
// kSleepNs > 0 puts the warp to sleep between polls.  A polling warp is always ready to issue, so it takes issue
// slots from the warps that share its scheduler; only a wait whose wake-up latency is on the critical path (the MMA
// issuer's) should poll without sleeping.
template <int kSleepNs = 0>
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int where) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    for (int i = 0; i < 128; ++i) {
      if (kSleepNs > 0) __nanosleep(kSleepNs);
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitLimitCycles) {
      *abort_flag = 1;
      dsv4_set_error(DSV4_ERR_WAIT_TIMEOUT, where, (int)blockIdx.x);
      return false;
    }
  }
}

// ---------------------------------------------------------------- programmatic dependent launch
// Every kernel of this library is launched with the programmatic-stream-serialization attribute: it may start while
// the kernel before it in the stream is still running, which hides launch latency and the prologue (barrier init,
// tensor-memory allocation, weight prefetch).  pdl_wait() blocks until every earlier kernel has completed and its
// memory is visible; no kernel touches data of an earlier kernel before it.  pdl_launch_dependents() lets the next
// kernel start.
//
// A kernel lets its successor start only AFTER its own wait, never before.  With the trigger first, a chain of
// kernels runs ahead several deep: a kernel's CTAs can already sit on an SM while kernels two and three places
// earlier still run there.  Loads through the read-only path (what `const __restrict__` compiles to) then hit lines
// that an earlier kernel's CTA brought into that SM's L1 after the late kernel's start, and when the allocator has
// meanwhile handed the address to a new tensor, the late kernel reads the old tensor's bytes: seen as a route plan
// header that held the router's scores, in a captured graph where launches follow each other without host gaps.
// With the wait first, a kernel starts only once everything before its predecessor has completed.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_entry() {
  pdl_wait();
  pdl_launch_dependents();
}

// ---------------------------------------------------------------- thread-block clusters
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// barrier over every thread of every CTA of the cluster (all threads of a warp must call it together)
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// 16-byte load from the shared memory of CTA `rank` of the cluster, at the same offset as local address `addr`
__device__ __forceinline__ float4 ld_dsmem_f4(uint32_t addr, uint32_t rank) {
  uint32_t ra;
  float4 v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(addr), "r"(rank));
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(ra)
               : "memory");
  return v;
}

// ---------------------------------------------------------------- TMA
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int x, int y,
                                            int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::
          "r"(smem_u32(smem_dst)),
      "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}
// generic-proxy smem writes -> visible to the async proxy (TMA / tcgen05 reads)
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------- tcgen05 / TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_holder, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_holder)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// commit all previously issued tcgen05.mma of this thread; the mbarrier gets one arrival when they finish
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// D[tmem] (+)= A[smem] * B[smem];  kind::f16 covers fp16/bf16 inputs, kind::f8f6f4 the 8/6/4-bit float inputs
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]: the A operand sits in tensor memory, row i of the 128-row tile on lane i and the
// K elements packed two per 32-bit column (16-bit types), so K = 16 of one instruction spans 8 columns.
__device__ __forceinline__ void umma_f16_ta(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_f8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Shared-memory matrix descriptor for a K-major tile whose rows are exactly one
// 128-byte swizzle span (64 bf16 or 128 fp8) and packed 128 B apart: 8-row
// groups are 1024 B apart (SBO), the tile base is 1024-B aligned, version = 1.
__device__ __forceinline__ uint64_t umma_desc_k128(const void* smem_tile, uint32_t byte_offset_in_row) {
  uint32_t addr = smem_u32(smem_tile) + byte_offset_in_row;
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);          // start address, bits [0,14)
  d |= (uint64_t)1 << 16;                          // LBO (unused for swizzled K-major), bits [16,30)
  d |= (uint64_t)(1024 >> 4) << 32;                // SBO = 1024 B, bits [32,46)
  d |= (uint64_t)1 << 46;                          // descriptor version 1 (Blackwell)
  d |= (uint64_t)2 << 61;                          // SWIZZLE_128B
  return d;
}

// Instruction descriptor: fp32 accumulate, A and B both K-major.
// fmt: kind::f16 -> 0 = fp16, 1 = bf16;  kind::f8f6f4 -> 0 = e4m3, 1 = e5m2, 5 = e2m1
__host__ __device__ constexpr uint32_t umma_idesc(int M, int N, int a_fmt, int b_fmt) {
  return (1u << 4) | ((uint32_t)a_fmt << 7) | ((uint32_t)b_fmt << 10) | ((uint32_t)(N >> 3) << 17) |
         ((uint32_t)(M >> 4) << 24);
}

// ---- block-scaled MMA (kind::mxf8f6f4): D (+)= (A * SFA) (B * SFB), one ue8m0 scale per row and 32 K elements.
// Instruction descriptor: a_fmt / b_fmt as for kind::f8f6f4, scale format e8m0, fp32 accumulate, both operands K-major.
// The instruction covers K = 32; its scales are byte `sf_id` (0..3) of the 32-bit tensor-memory cells at sfa / sfb.
__host__ __device__ constexpr uint32_t umma_idesc_mx(int M, int N, int a_fmt, int b_fmt) {
  return ((uint32_t)a_fmt << 7) | ((uint32_t)b_fmt << 10) | ((uint32_t)(N >> 3) << 17) | (1u << 23) |
         ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void umma_mx(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sf_id,
                                        uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  const uint32_t id = idesc | (sf_id << 4) | (sf_id << 29);
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(id), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
// Scale factors of 128 rows x 4 K blocks: 512 contiguous bytes of shared memory, byte (row % 32) * 16 + (row / 32) * 4
// + block.  The copy puts them into 4 tensor-memory columns (lane = row % 32 in each of the four 32-lane groups,
// column = row / 32, byte = block), the arrangement the block-scaled MMA reads.  It is ordered after the MMAs this
// thread issued before it and before those it issues afterwards.
__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, const void* smem_sf) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_u32(smem_sf) & 0x3FFFF) >> 4);  // 32 rows of 16 bytes, no swizzle
  d |= (uint64_t)1 << 16;                               // LBO (one 16-byte column: unused)
  d |= (uint64_t)(128 >> 4) << 32;                      // SBO: 8-row groups are 128 B apart
  d |= (uint64_t)1 << 46;
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(d) : "memory");
}
// untiled bulk copy global -> shared, completion counted on an mbarrier (both addresses and the size multiples of 16)
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// 32 lanes x 32 consecutive fp32 columns: thread t of the warp gets row (lane base + t)
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// registers -> TMEM: thread (lane) i of the warp writes 16 consecutive 32-bit columns of TMEM lane (warp % 4) * 32 + i
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------- misc math
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float bf2f(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ __nv_bfloat16 f2bf(float v) { return __float2bfloat16_rn(v); }

// ---------------------------------------------------------------- FP8 activation quantisation (shared by the fused producers)
// scale = 2^ceil(log2(max(absmax, 1e-4) / 448)); q = e4m3_rn(clamp(x / scale)), one scale per (row, 128 columns)
__device__ __forceinline__ float pow2_ceil_scale(float amax) {
  const float v = __fdiv_rn(fmaxf(amax, 1e-4f), 448.f);
  const uint32_t b = __float_as_uint(v);
  int e = (int)((b >> 23) & 0xff) - 127 + ((b & 0x7fffff) ? 1 : 0);
  return __uint_as_float((uint32_t)(e + 127) << 23);
}
// v: 8 consecutive (already bf16-rounded) values of one row starting at column `col` (a multiple of 8).  The 16
// lanes that share (lane / 16) hold one 128-column block; every lane of the warp must call this together.
__device__ __forceinline__ void quant8_store(const float (&v)[8], uint8_t* __restrict__ qrow, float* __restrict__ srow,
                                             int col) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
  for (int o = 1; o < 16; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float sc = pow2_ceil_scale(amax);
  const float inv = 1.f / sc;  // exact: power of two
  uint32_t w[2] = {0, 0};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float c = fminf(fmaxf(v[i] * inv, -448.f), 448.f);
    w[i >> 2] |= (uint32_t)__nv_cvt_float_to_fp8(c, __NV_SATFINITE, __NV_E4M3) << (8 * (i & 3));
  }
  *reinterpret_cast<uint2*>(qrow + col) = make_uint2(w[0], w[1]);
  if ((threadIdx.x & 15) == 0) srow[col >> 7] = sc;
}

// host side -----------------------------------------------------------------
// Launches `kernel` with programmatic dependent launch allowed (set DSV4_PDL=0 in the environment to launch plainly).
bool dsv4_pdl_enabled();
template <typename... KArgs, typename... Args>
inline cudaError_t dsv4_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                               Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dsv4_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
// Same, with the CTAs grouped into clusters of `cluster_z` along grid.z.
template <typename... KArgs, typename... Args>
inline cudaError_t dsv4_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                       int cluster_z, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = cluster_z;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dsv4_pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Encodes a 2-D row-major tensor map (inner = contiguous dimension) with the given box and swizzle.
// Returns 0 on success.  elem: 0 = uint8, 1 = bf16, 2 = fp32, 3 = packed 4-bit values that land in shared memory
// as 16 values per 16 bytes (8 bytes of nibbles, 8 bytes of gap: the operand form of the f8f6f4 MMA kinds; inner,
// box_inner count 4-bit elements, box_inner must be 128, base and row stride multiples of 32 bytes).
// swizzle: 0 = none, 3 = 128 B.
int dsv4_make_tmap_2d(CUtensorMap* out, const void* base, int elem, uint64_t inner, uint64_t outer,
                      uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, int swizzle);
