// Fused GEMM epilogue shared by the tensor-core and SIMT projection kernels:
//   v = acc; v += bias[n]; act; v *= gate_b[n]; v += residual[m, n]
#pragma once
#include "common.cuh"

namespace sana {

struct EpiParams {
  const void* bias;
  const void* gate_table;
  const void* gate_t;
  const void* residual;
  int64_t ldr;
  int64_t rows_per_batch;
  int64_t relu_cols;
  int32_t act;
  int32_t gate_row;
};

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// exact SiLU for the fp32 path, fast intrinsics for bf16 outputs
template <typename T>
__device__ __forceinline__ float epi_silu(float x);
template <>
__device__ __forceinline__ float epi_silu<float>(float x) { return x / (1.0f + expf(-x)); }
template <>
__device__ __forceinline__ float epi_silu<__nv_bfloat16>(float x) { return silu(x); }

// GELU, tanh form (nn.GELU(approximate="tanh")): 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))
__device__ __forceinline__ float gelu_tanh(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.0f + tanhf(u));
}

// scalar form (SIMT kernel)
template <typename T>
__device__ __forceinline__ float epi_scalar(float v, int64_t m, int64_t n, int64_t N, const EpiParams& p) {
  if (p.bias) v += to_f32(static_cast<const T*>(p.bias)[n]);
  if (p.act == 1) v = epi_silu<T>(v);
  else if (p.act == 2 && n < p.relu_cols) v = fmaxf(v, 0.f);
  else if (p.act == 3) v = gelu_tanh(v);
  if (p.gate_table) {
    const int64_t b = m / p.rows_per_batch;
    const float g = to_f32(static_cast<const T*>(p.gate_table)[(int64_t)p.gate_row * N + n]) +
                    to_f32(static_cast<const T*>(p.gate_t)[(b * 6 + p.gate_row) * N + n]);
    v *= g;
  }
  if (p.residual) v += to_f32(static_cast<const T*>(p.residual)[m * p.ldr + n]);
  return v;
}

// 8 consecutive bf16 columns n .. n+7 of row m (tensor-core kernel); n is a multiple of 8.
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  f[0] = bf16_lo(u.x), f[1] = bf16_hi(u.x), f[2] = bf16_lo(u.y), f[3] = bf16_hi(u.y);
  f[4] = bf16_lo(u.z), f[5] = bf16_hi(u.z), f[6] = bf16_lo(u.w), f[7] = bf16_hi(u.w);
}

__device__ __forceinline__ uint4 epi_vec8_bf16(float (&v)[8], int64_t m, int64_t n, int64_t N, int64_t batch,
                                               const EpiParams& p) {
  float f[8];
  if (p.bias) {
    unpack8(__ldg(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.bias) + n)), f);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] += f[e];
  }
  if (p.act == 1) {
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = silu(v[e]);
  } else if (p.act == 2) {
#pragma unroll
    for (int e = 0; e < 8; ++e)
      if (n + e < p.relu_cols) v[e] = fmaxf(v[e], 0.f);
  } else if (p.act == 3) {
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = gelu_tanh(v[e]);
  }
  if (p.gate_table) {
    float g[8];
    unpack8(__ldg(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.gate_table) +
                                                  (int64_t)p.gate_row * N + n)), g);
    unpack8(__ldg(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.gate_t) +
                                                  (batch * 6 + p.gate_row) * N + n)), f);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] *= (g[e] + f[e]);
  }
  if (p.residual) {
    unpack8(ldg_nc_u4(static_cast<const __nv_bfloat16*>(p.residual) + m * p.ldr + n), f);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] += f[e];
  }
  return make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
}

inline int check_epilogue(const sana_gemm_epilogue* ep, int64_t N, EpiParams* out, const char* who) {
  EpiParams p{};
  p.rows_per_batch = 1;
  if (ep) {
    p.bias = ep->bias;
    p.gate_table = ep->gate_table;
    p.gate_t = ep->gate_t;
    p.residual = ep->residual;
    p.ldr = ep->ldr;
    p.rows_per_batch = ep->rows_per_batch;
    p.relu_cols = ep->relu_cols;
    p.act = ep->act;
    p.gate_row = ep->gate_row;
    if (p.act < 0 || p.act > 3) return fail(SANA_ERR_INVALID, "%s: act must be 0, 1, 2 or 3", who);
    if (p.gate_table) {
      if (!p.gate_t) return fail(SANA_ERR_INVALID, "%s: gate_t required with gate_table", who);
      if (p.gate_row < 0 || p.gate_row > 5) return fail(SANA_ERR_INVALID, "%s: gate_row out of range", who);
      if (p.rows_per_batch <= 0) return fail(SANA_ERR_INVALID, "%s: rows_per_batch must be positive", who);
    } else {
      p.rows_per_batch = 1;
    }
    if (p.residual && p.ldr < N) return fail(SANA_ERR_INVALID, "%s: ldr < N", who);
  }
  *out = p;
  return SANA_OK;
}

}  // namespace sana
