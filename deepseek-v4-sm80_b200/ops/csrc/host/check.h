// Host-side argument checking shared by the C++ helpers.
//
// A `Check` collects the first failed condition with the source location and a
// formatted message; exported functions return its code instead of throwing
// across the C ABI.  It plays the role of the reference's RuntimeCheck/panic
// helpers (python/minisgl/kernel/csrc/include/minisgl/utils.h:40-92) and of its
// declarative tensor matcher (include/minisgl/tensor.h:140-300): here a tensor
// is described by a small POD view and verified field by field.
#pragma once
#include <cstdint>
#include <cstdio>
#include <source_location>
#include <string>

#define DSV4_HOST_API extern "C" __attribute__((visibility("default")))

namespace dsv4 {

struct TensorView {
  const void* data;
  int64_t shape[4];
  int64_t stride[4];  // in elements
  int32_t ndim;
  int32_t dtype;   // 0 u8, 1 bf16, 2 f32, 3 i32, 4 i64, 5 fp8e4m3
  int32_t device;  // -1 cpu, >=0 cuda ordinal
};

inline thread_local std::string g_last_error;

class Check {
 public:
  bool ok() const { return ok_; }
  Check& require(bool cond, const char* what, std::source_location loc = std::source_location::current()) {
    if (ok_ && !cond) {
      ok_ = false;
      char buf[512];
      std::snprintf(buf, sizeof buf, "%s:%u: check failed: %s", loc.file_name(), (unsigned)loc.line(), what);
      g_last_error = buf;
    }
    return *this;
  }
  Check& dim(const TensorView& t, int expect, const char* name) {
    return require(t.ndim == expect, name);
  }
  Check& dtype(const TensorView& t, int expect, const char* name) { return require(t.dtype == expect, name); }
  Check& contiguous(const TensorView& t, const char* name) {
    int64_t s = 1;
    bool c = true;
    for (int i = t.ndim - 1; i >= 0; --i) {
      if (t.shape[i] != 1 && t.stride[i] != s) c = false;
      s *= t.shape[i];
    }
    return require(c, name);
  }
  Check& same_device(const TensorView& a, const TensorView& b, const char* name) {
    return require(a.device == b.device, name);
  }

 private:
  bool ok_ = true;
};

}  // namespace dsv4
