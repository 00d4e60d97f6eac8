// Library-wide state: the device status word, tensor-map encoding, version probe.
#include "common.cuh"

#include <cstdlib>

#include <stdio.h>
#include <string.h>

__device__ int g_dsv4_status[8];
__device__ unsigned long long g_dsv4_peer_wait_ns = 2000000000ull;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

int dsv4_make_tmap_2d(CUtensorMap* out, const void* base, int elem, uint64_t inner, uint64_t outer,
                      uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, int swizzle) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return 1;
  CUtensorMapDataType dt = elem == 0   ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                           : elem == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : elem == 3 ? CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B
                                       : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapSwizzle sw = swizzle == 3   ? CU_TENSOR_MAP_SWIZZLE_128B
                          : swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_64B
                          : swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_32B
                                         : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 2;
}

// Copies the 8-int status word to `host_out` (synchronises the device) and optionally clears it.
DSV4_API int dsv4_read_status(int* host_out, int clear) {
  cudaError_t e = cudaMemcpyFromSymbol(host_out, g_dsv4_status, sizeof(int) * 8);
  if (e != cudaSuccess) return (int)e;
  if (clear) {
    int z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    e = cudaMemcpyToSymbol(g_dsv4_status, z, sizeof(z));
  }
  return (int)e;
}

// Queues a copy of the status word into `pinned_host` (8 ints of page-locked host memory) on `st`, without
// synchronising: the caller reads it after whatever it already waits for on that stream.  A serving loop uses this
// once per step, so that a wait that ran out on the device becomes a host error within one step.
DSV4_API int dsv4_status_snapshot(int* pinned_host, cudaStream_t st) {
  void* sym = nullptr;
  cudaError_t e = cudaGetSymbolAddress(&sym, g_dsv4_status);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemcpyAsync(pinned_host, sym, sizeof(int) * 8, cudaMemcpyDeviceToHost, st);
}

// Sets the limit of waits on other GPUs (current device).  Values below 1 ms are refused.
DSV4_API int dsv4_set_peer_wait_ms(long long ms) {
  if (ms < 1) return 1;
  const unsigned long long ns = (unsigned long long)ms * 1000000ull;
  return (int)cudaMemcpyToSymbol(g_dsv4_peer_wait_ns, &ns, sizeof(ns));
}

bool dsv4_pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("DSV4_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}

DSV4_API int dsv4_abi_version() { return 1; }
