// RMSNorm over the channel dimension with a learned weight (the optional q/k normalisation of
// the attention layers): y = weight * x * rsqrt(mean(x^2) + eps), statistics in fp32, one
// rounding on store.  One warp per row, the row held packed in registers; input and output may
// be column slices of wider tensors (row strides in elements) and may alias (in place).
#include "common.cuh"

namespace sana {

template <int MAXV>
__global__ void __launch_bounds__(256)
rmsnorm_bf16_kernel(const __nv_bfloat16* x, int64_t ldx, const __nv_bfloat16* __restrict__ w, __nv_bfloat16* y,
                    int64_t ldy, int64_t rows, int C, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nvec = C >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * ldx);
  uint4 raw[MAXV];
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = lane + 32 * i;
    if (v < nvec) {
      raw[i] = xr[v];
      const uint32_t wd[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float a = bf16_lo(wd[e]), b = bf16_hi(wd[e]);
        sq = fmaf(a, a, sq);
        sq = fmaf(b, b, sq);
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
  const float r = rsqrtf(sq / (float)C + eps);
  uint4* yr = reinterpret_cast<uint4*>(y + row * ldy);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = lane + 32 * i;
    if (v < nvec) {
      const uint4 wv = __ldg(wr + v);
      const uint32_t xd[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
      const uint32_t wd[4] = {wv.x, wv.y, wv.z, wv.w};
      uint32_t o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e)
        o[e] = pack_bf16(bf16_lo(wd[e]) * (bf16_lo(xd[e]) * r), bf16_hi(wd[e]) * (bf16_hi(xd[e]) * r));
      yr[v] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// fp32 parity path: one thread block per row
__global__ void __launch_bounds__(256)
rmsnorm_f32_kernel(const float* x, int64_t ldx, const float* __restrict__ w, float* y, int64_t ldy, int C, float eps) {
  __shared__ float red[8];
  const float* xr = x + (int64_t)blockIdx.x * ldx;
  float* yr = y + (int64_t)blockIdx.x * ldy;
  float sq = 0.f;
  for (int c = threadIdx.x; c < C; c += 256) sq = fmaf(xr[c], xr[c], sq);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float r = rsqrtf(tot / (float)C + eps);
  for (int c = threadIdx.x; c < C; c += 256) yr[c] = w[c] * (xr[c] * r);
}

}  // namespace sana

using namespace sana;

extern "C" int sana_rmsnorm(const void* x, int64_t ldx, const void* weight, void* y, int64_t ldy, int64_t rows,
                            int64_t C, float eps, int dtype, void* stream) {
  SANA_REQUIRE(x && weight && y, "sana_rmsnorm: null pointer");
  SANA_REQUIRE(rows > 0 && C > 0 && C % 8 == 0 && C <= 8192, "sana_rmsnorm: C must be a positive multiple of 8, at most 8192");
  SANA_REQUIRE(ldx >= C && ldy >= C && ldx % 8 == 0 && ldy % 8 == 0, "sana_rmsnorm: row strides must be >= C and multiples of 8");
  SANA_REQUIRE(aligned16(x) && aligned16(y) && aligned16(weight), "sana_rmsnorm: pointers must be 16-byte aligned");
  SANA_REQUIRE(rows < ((int64_t)1 << 31), "sana_rmsnorm: too many rows");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == SANA_BF16) {
    const int per_lane = (int)ceil_div(C / 8, 32);
    const unsigned grid = (unsigned)ceil_div(rows, 8);
    const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
    const __nv_bfloat16* wp = static_cast<const __nv_bfloat16*>(weight);
    __nv_bfloat16* yp = static_cast<__nv_bfloat16*>(y);
    if (per_lane <= 5) rmsnorm_bf16_kernel<5><<<grid, 256, 0, st>>>(xp, ldx, wp, yp, ldy, rows, (int)C, eps);
    else if (per_lane <= 9) rmsnorm_bf16_kernel<9><<<grid, 256, 0, st>>>(xp, ldx, wp, yp, ldy, rows, (int)C, eps);
    else if (per_lane <= 16) rmsnorm_bf16_kernel<16><<<grid, 256, 0, st>>>(xp, ldx, wp, yp, ldy, rows, (int)C, eps);
    else rmsnorm_bf16_kernel<32><<<grid, 256, 0, st>>>(xp, ldx, wp, yp, ldy, rows, (int)C, eps);
  } else if (dtype == SANA_F32) {
    rmsnorm_f32_kernel<<<(unsigned)rows, 256, 0, st>>>(static_cast<const float*>(x), ldx, static_cast<const float*>(weight),
                                                       static_cast<float*>(y), ldy, (int)C, eps);
  } else {
    return fail(SANA_ERR_UNSUPPORTED, "sana_rmsnorm: unsupported dtype %d", dtype);
  }
  SANA_LAUNCH_CHECK("rmsnorm kernel");
  return SANA_OK;
}

// ------------------------------------------------------------------------------------------
// Rotary embedding on the q or k column block of a qkv projection, in place, before the ReLU
// feature map: channel pairs (2i, 2i+1) of every 32-channel head are rotated with per-position
// tables, y = x * cos + rot(x) * sin with rot(x)[2i] = -x[2i+1], rot(x)[2i+1] = x[2i]; fp32
// arithmetic, one rounding on store.  One thread per channel pair.
// ------------------------------------------------------------------------------------------
namespace sana {

template <typename T>
__device__ __forceinline__ float rope_ld(const T* p);
template <>
__device__ __forceinline__ float rope_ld<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float rope_ld<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T>
__device__ __forceinline__ void rope_st(T* p, float v);
template <>
__device__ __forceinline__ void rope_st<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void rope_st<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

template <typename T>
__global__ void rope_kernel(T* x, int64_t ld, const float* __restrict__ cosv, const float* __restrict__ sinv,
                            int64_t rows, int N, int C, int D) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int half = C >> 1;
  if (idx >= rows * half) return;
  const int64_t row = idx / half;
  const int c = (int)(idx - row * half) * 2;  // even channel of the pair
  const int d = c % D;                       // position inside the head
  const int64_t pos = row % N;
  T* px = x + row * ld + c;
  const float a = rope_ld(px), b = rope_ld(px + 1);
  const float* cr = cosv + pos * D + d;
  const float* sr = sinv + pos * D + d;
  rope_st(px, a * cr[0] + (-b) * sr[0]);
  rope_st(px + 1, b * cr[1] + a * sr[1]);
}

}  // namespace sana

extern "C" int sana_rope(void* x, int64_t ld, const float* cos_table, const float* sin_table, int64_t B, int64_t N,
                         int64_t C, int64_t head_dim, int dtype, void* stream) {
  SANA_REQUIRE(x && cos_table && sin_table, "sana_rope: null pointer");
  SANA_REQUIRE(B > 0 && N > 0 && C > 0 && head_dim > 0, "sana_rope: sizes must be positive");
  SANA_REQUIRE(head_dim % 2 == 0 && C % head_dim == 0, "sana_rope: C must be whole heads of an even dimension");
  SANA_REQUIRE(ld >= C && N < ((int64_t)1 << 31) && C < ((int64_t)1 << 30), "sana_rope: bad stride or size");
  const int64_t total = B * N * (C / 2);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)ceil_div(total, 256);
  if (dtype == SANA_BF16)
    rope_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<__nv_bfloat16*>(x), ld, cos_table, sin_table, B * N,
                                                    (int)N, (int)C, (int)head_dim);
  else if (dtype == SANA_F32)
    rope_kernel<float><<<grid, 256, 0, st>>>(static_cast<float*>(x), ld, cos_table, sin_table, B * N, (int)N, (int)C,
                                            (int)head_dim);
  else
    return fail(SANA_ERR_UNSUPPORTED, "sana_rope: unsupported dtype %d", dtype);
  SANA_LAUNCH_CHECK("rope kernel");
  return SANA_OK;
}
