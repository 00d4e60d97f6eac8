// Sparse MQA attention over the paged caches: per token, all local heads attend
//   {sink} U {selected C4 rows | all C128 rows | nothing} U {sliding window rows},
// keys and values being the same 512-d latent row (K = V), softmax scale 512^-1/2.
// One CTA per token: every gathered row is fetched once (cp.async, double buffered, 32 rows per tile) and
// shared by all local heads.  The kernel walks the request's page-table row itself, so no index surface is
// materialised: compressed entry j of ratio r lives at row comp_row(page_table[slot, j*r + r-1]); window position
// p lives at swa_map[loc / ps] * ps + loc % ps.  (m, l) start at (sink, 1), which adds exp(sink - m) to the
// denominator only -- the reference's two-source kernel semantics
// (python/minisgl/kernel/csrc/jit/dsv4_sparse_attention_two_source_bf16.cu:77-168).
#include "common.cuh"

namespace {

constexpr int D = 512;
constexpr int KT = 32;  // keys per tile
constexpr int NTHR = 256;

__device__ __forceinline__ void cp_async16(void* smem, const void* g) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem)), "l"(g) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
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
};

template <int HL>
__global__ void __launch_bounds__(NTHR) sparse_attn_kernel(AttnArgs a) {
  extern __shared__ __align__(16) uint8_t attn_smem[];
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(attn_smem);            // [HL][D]
  __nv_bfloat16* kvs = qs + HL * D;                                           // [2][KT][D]
  float* ps_ = reinterpret_cast<float*>(kvs + 2 * KT * D);                    // [HL][KT] probabilities
  float* alpha = ps_ + HL * KT;                                               // [HL]
  float* ms = alpha + HL;                                                     // [HL]
  float* ls = ms + HL;                                                        // [HL]
  int* valid = reinterpret_cast<int*>(ls + HL);                               // [2][KT]

  const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (a.num_valid && t >= *a.num_valid) {
    for (int i = tid; i < HL * D / 8; i += NTHR) reinterpret_cast<uint4*>(a.o + (size_t)t * HL * D)[i] = make_uint4(0, 0, 0, 0);
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

  for (int i = tid; i < HL * D / 8; i += NTHR)
    reinterpret_cast<uint4*>(qs)[i] = reinterpret_cast<const uint4*>(a.q + (size_t)t * HL * D)[i];
  if (tid < HL) ms[tid] = a.sink[tid], ls[tid] = 1.f;

  auto issue_tile = [&](int tile, int buf) {
    const int key = tile * KT + (tid >> 3);
    const __nv_bfloat16* src = nullptr;
    if (key < ntot) {
      if (key < nc) {
        const int j = a.mode == 1 ? a.topk_idx[(size_t)t * a.topk_width + key] : key;
        if (j >= 0) {
          const int loc = pt[j * a.ratio + a.ratio - 1];
          src = a.comp + ((size_t)(loc / a.ps) * rpp + (loc % a.ps) / a.ratio) * D;
        }
      } else {
        const int pp = p - ns + 1 + (key - nc);
        const int loc = pt[pp];
        const int ss = a.swa_map[loc / a.ps];
        if (ss >= 0) src = a.swa + ((size_t)ss * a.ps + loc % a.ps) * D;
      }
    }
    __nv_bfloat16* dst = kvs + ((size_t)buf * KT + (tid >> 3)) * D;
    if (src) {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const int ch = (tid & 7) + 8 * c;
        cp_async16(dst + ch * 8, src + ch * 8);
      }
    }
    if ((tid & 7) == 0) valid[buf * KT + (tid >> 3)] = src != nullptr;
    cp_async_commit();
  };

  float acc[HL][2];
#pragma unroll
  for (int h = 0; h < HL; ++h) acc[h][0] = acc[h][1] = 0.f;

  if (ntiles > 0) issue_tile(0, 0);
  for (int tile = 0; tile < ntiles; ++tile) {
    const int buf = tile & 1;
    if (tile + 1 < ntiles) {
      issue_tile(tile + 1, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const __nv_bfloat16* kt = kvs + (size_t)buf * KT * D;
    // scores: warp w handles keys w, w+8, w+16, w+24; lane holds 16 dims of the key in registers
#pragma unroll 1
    for (int kk = warp; kk < KT; kk += 8) {
      const bool ok = valid[buf * KT + kk] != 0;
      float kf[16];
      if (ok) {
        const uint4 u0 = *reinterpret_cast<const uint4*>(kt + kk * D + lane * 16);
        const uint4 u1 = *reinterpret_cast<const uint4*>(kt + kk * D + lane * 16 + 8);
        const __nv_bfloat162* p0 = reinterpret_cast<const __nv_bfloat162*>(&u0);
        const __nv_bfloat162* p1 = reinterpret_cast<const __nv_bfloat162*>(&u1);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f0 = __bfloat1622float2(p0[i]), f1 = __bfloat1622float2(p1[i]);
          kf[2 * i] = f0.x, kf[2 * i + 1] = f0.y, kf[8 + 2 * i] = f1.x, kf[8 + 2 * i + 1] = f1.y;
        }
      }
      for (int h = 0; h < HL; ++h) {
        float s = 0.f;
        if (ok) {
          const uint4 u0 = *reinterpret_cast<const uint4*>(qs + h * D + lane * 16);
          const uint4 u1 = *reinterpret_cast<const uint4*>(qs + h * D + lane * 16 + 8);
          const __nv_bfloat162* p0 = reinterpret_cast<const __nv_bfloat162*>(&u0);
          const __nv_bfloat162* p1 = reinterpret_cast<const __nv_bfloat162*>(&u1);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f0 = __bfloat1622float2(p0[i]), f1 = __bfloat1622float2(p1[i]);
            s = fmaf(f0.x, kf[2 * i], s);
            s = fmaf(f0.y, kf[2 * i + 1], s);
            s = fmaf(f1.x, kf[8 + 2 * i], s);
            s = fmaf(f1.y, kf[8 + 2 * i + 1], s);
          }
          s = warp_sum(s);
        }
        if (lane == 0) ps_[h * KT + kk] = ok ? s * a.scale : -INFINITY;
      }
    }
    __syncthreads();
    // online softmax bookkeeping: one thread per head
    if (tid < HL) {
      float m_old = ms[tid], mx = m_old;
#pragma unroll
      for (int k = 0; k < KT; ++k) mx = fmaxf(mx, ps_[tid * KT + k]);
      float sum = 0.f;
#pragma unroll
      for (int k = 0; k < KT; ++k) {
        const float e = __expf(ps_[tid * KT + k] - mx);
        ps_[tid * KT + k] = e;
        sum += e;
      }
      const float al = __expf(m_old - mx);
      alpha[tid] = al;
      ms[tid] = mx;
      ls[tid] = ls[tid] * al + sum;
    }
    __syncthreads();
    // O += P V ; thread owns dims {2*tid, 2*tid+1} of every head
#pragma unroll
    for (int h = 0; h < HL; ++h) {
      const float al = alpha[h];
      acc[h][0] *= al;
      acc[h][1] *= al;
    }
#pragma unroll 4
    for (int k = 0; k < KT; ++k) {
      if (!valid[buf * KT + k]) continue;
      const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(kt + k * D + 2 * tid));
#pragma unroll
      for (int h = 0; h < HL; ++h) {
        const float pv = ps_[h * KT + k];
        acc[h][0] = fmaf(pv, v.x, acc[h][0]);
        acc[h][1] = fmaf(pv, v.y, acc[h][1]);
      }
    }
    __syncthreads();
  }
  __syncthreads();
#pragma unroll
  for (int h = 0; h < HL; ++h) {
    const float inv = 1.f / ls[h];
    *reinterpret_cast<__nv_bfloat162*>(a.o + ((size_t)t * HL + h) * D + 2 * tid) =
        __floats2bfloat162_rn(acc[h][0] * inv, acc[h][1] * inv);
  }
}

template <int HL>
int launch_attn(const AttnArgs& a, int t, cudaStream_t st) {
  const int smem = HL * D * 2 + 2 * KT * D * 2 + (HL * KT + 3 * HL) * 4 + 2 * KT * 4;
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(sparse_attn_kernel<HL>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return 301;
    set = true;
  }
  sparse_attn_kernel<HL><<<t, NTHR, smem, st>>>(a);
  return (int)cudaGetLastError();
}

}  // namespace

DSV4_API int dsv4_sparse_attention(const void* q, void* o, const int* slots, const int* pos, const int* page_table,
                                   int ld_pt, const void* swa, const int* swa_map, const void* comp,
                                   const int* topk_idx, const int* topk_len, int topk_width, int mode, int ratio,
                                   const float* sink, float scale, int ps, int window, const int* num_valid, int t,
                                   int heads, int d, cudaStream_t st) {
  if (t <= 0) return 0;
  if (d != D) return 300;
  AttnArgs a{(const __nv_bfloat16*)q, (__nv_bfloat16*)o, slots, pos, page_table, ld_pt, (const __nv_bfloat16*)swa,
             swa_map, (const __nv_bfloat16*)comp, topk_idx, topk_len, topk_width, mode, ratio, sink, scale, ps,
             window, num_valid};
  switch (heads) {
    case 8: return launch_attn<8>(a, t, st);
    case 16: return launch_attn<16>(a, t, st);
    case 32: return launch_attn<32>(a, t, st);
    case 64: return launch_attn<64>(a, t, st);
    default: return 302;
  }
}
