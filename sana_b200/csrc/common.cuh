// Shared device/host helpers for the Linear-DiT block kernels (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/sana_b200.h"

namespace sana {

// ---- host-side status plumbing -----------------------------------------------------------
// Records a message retrievable through sana_last_error() and returns `code`.
int fail(int code, const char* fmt, ...);

inline int cuda_status(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return SANA_OK;
  return fail(static_cast<int>(e), "%s: %s", what, cudaGetErrorString(e));
}

#define SANA_REQUIRE(cond, ...)                                   \
  do {                                                            \
    if (!(cond)) return ::sana::fail(SANA_ERR_INVALID, __VA_ARGS__); \
  } while (0)

#define SANA_LAUNCH_CHECK(name) \
  do {                          \
    cudaError_t e__ = cudaGetLastError(); \
    if (e__ != cudaSuccess) return ::sana::cuda_status(e__, name); \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

int sm_count();  // SMs of the current device (cached per device)

// Limit, in nanoseconds, of the waits for a peer GPU inside the sequence-parallel exchange
// kernels (process-wide; set by sana_exchange_set_wait_limit_ns, 2 s unless changed).
long long exchange_wait_limit_ns();

// One flag per device for set-up that must happen once on every device the process uses
// (function attributes live in a device's context).  A lost race repeats harmless work.
struct OncePerDevice {
  bool done[64] = {};
  bool first_time() {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= 64) return true;
    if (done[d]) return false;
    done[d] = true;
    return true;
  }
};

// ---- small device helpers -------------------------------------------------------------------
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&r);
}

__device__ __forceinline__ uint32_t relu_bf16x2(uint32_t v) {
  __nv_bfloat162 x = *reinterpret_cast<__nv_bfloat162*>(&v);
  x = __hmax2(x, __floats2bfloat162_rn(0.f, 0.f));
  return *reinterpret_cast<uint32_t*>(&x);
}

__device__ __forceinline__ float silu(float x) { return x * __frcp_rn(1.0f + __expf(-x)); }

// two fp32 FMAs in one instruction (sm_100 packed fp32 pipe)
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }

// warp-level bf16 tensor-core product, fp32 accumulate: D(16x8) += A(16x16) * B(16x8)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint2 ldg_nc_u2(const void* p) {
  uint2 r;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p));
  return r;
}
__device__ __forceinline__ uint4 ldg_nc_u4(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

}  // namespace sana
