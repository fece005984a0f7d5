// The small steps either side of the block loop of the DiT forward: latent <-> token layout
// changes (patchify / unpatchify), the sinusoidal timestep features and an elementwise SiLU.
// All of them move a few MB at most; they exist so that the whole forward runs on this
// library's kernels.
#include <cmath>

#include "common.cuh"

namespace sana {

template <typename T>
__device__ __forceinline__ float ld_f32(const T* p);
template <>
__device__ __forceinline__ float ld_f32<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ld_f32<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T>
__device__ __forceinline__ void st_f32(T* p, float v);
template <>
__device__ __forceinline__ void st_f32<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void st_f32<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// patches[b, hp*Wp + wp, (c*p + i)*p + j] = x[b, c, hp*p + i, wp*p + j]: the unfold that turns the
// stride-p, kernel-p patch convolution into a projection with the conv weight viewed as
// [embed, Cin*p*p].  One thread per output element, consecutive threads along the patch row.
template <typename T>
__global__ void patchify_kernel(const T* __restrict__ x, T* __restrict__ out, int Cin, int H, int W, int p, int ld,
                                int64_t total) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int kk = Cin * p * p;
  const int e = (int)(idx % kk);
  const int64_t tok = idx / kk;
  const int Wp = W / p, Hp = H / p;
  const int wp = (int)(tok % Wp);
  const int hp = (int)((tok / Wp) % Hp);
  const int64_t b = tok / ((int64_t)Wp * Hp);
  const int j = e % p, i = (e / p) % p, c = e / (p * p);
  out[tok * ld + e] = x[((b * Cin + c) * H + hp * p + i) * (int64_t)W + wp * p + j];
}

// imgs[b, c, h*p + i, w*p + j] = tok[b, h*Wp + w, (i*p + j)*Cout + c]  ("nhwpqc->nchpwq")
template <typename T>
__global__ void unpatchify_kernel(const T* __restrict__ tok, T* __restrict__ out, int Cout, int Hp, int Wp, int p,
                                  int ld, int64_t total) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int W = Wp * p, H = Hp * p;
  const int xw = (int)(idx % W);
  const int yh = (int)((idx / W) % H);
  const int c = (int)((idx / ((int64_t)W * H)) % Cout);
  const int64_t b = idx / ((int64_t)W * H * Cout);
  const int w = xw / p, j = xw % p, h = yh / p, i = yh % p;
  out[idx] = tok[(b * Hp * Wp + (int64_t)h * Wp + w) * ld + (i * p + j) * Cout + c];
}

// out[b, :half] = cos(t_b * f_k), out[b, half:2*half] = sin(t_b * f_k), f_k = exp(-ln(max_period) k / half);
// an odd `dim` gets a trailing zero.  f_k and the product are rounded to fp32 as the reference
// computes them; exp, cos and sin are evaluated in double and rounded once.
template <typename T>
__global__ void timestep_embedding_kernel(const float* __restrict__ t, T* __restrict__ out, int B, int dim,
                                          float neg_log_period) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * dim) return;
  const int b = idx / dim, e = idx % dim;
  const int half = dim / 2;
  float v = 0.f;
  if (e < 2 * half) {
    const int k = e < half ? e : e - half;
    // the exponent is formed in fp32 as the reference forms it: (-ln(P) * k) / half
    const float expo = (neg_log_period * (float)k) / (float)half;
    const float f = (float)exp((double)expo);
    const float arg = t[b] * f;
    v = (float)(e < half ? cos((double)arg) : sin((double)arg));
  }
  st_f32(out + idx, v);
}

template <typename T>
__global__ void silu_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t n) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n) return;
  const float v = ld_f32(x + idx);
  st_f32(out + idx, v / (1.0f + expf(-v)));
}

}  // namespace sana

using namespace sana;

extern "C" int sana_patchify(const void* x, void* out, int64_t ldo, int64_t B, int64_t Cin, int64_t H, int64_t W,
                             int64_t p, int dtype, void* stream) {
  SANA_REQUIRE(x && out, "sana_patchify: null pointer");
  SANA_REQUIRE(B > 0 && Cin > 0 && H > 0 && W > 0 && p > 0, "sana_patchify: sizes must be positive");
  SANA_REQUIRE(H % p == 0 && W % p == 0, "sana_patchify: H and W must be multiples of the patch size");
  SANA_REQUIRE(ldo >= Cin * p * p, "sana_patchify: row stride smaller than a patch");
  SANA_REQUIRE(H < (1 << 20) && W < (1 << 20) && Cin * p * p < (1 << 24), "sana_patchify: size out of range");
  const int64_t total = B * (H / p) * (W / p) * Cin * p * p;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)ceil_div(total, 256);
  if (dtype == SANA_BF16)
    patchify_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x),
                                                        static_cast<__nv_bfloat16*>(out), (int)Cin, (int)H, (int)W,
                                                        (int)p, (int)ldo, total);
  else if (dtype == SANA_F32)
    patchify_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), static_cast<float*>(out), (int)Cin,
                                                (int)H, (int)W, (int)p, (int)ldo, total);
  else
    return fail(SANA_ERR_UNSUPPORTED, "sana_patchify: unsupported dtype %d", dtype);
  SANA_LAUNCH_CHECK("patchify kernel");
  return SANA_OK;
}

extern "C" int sana_unpatchify(const void* tok, int64_t ld, void* out, int64_t B, int64_t Cout, int64_t Hp, int64_t Wp,
                               int64_t p, int dtype, void* stream) {
  SANA_REQUIRE(tok && out, "sana_unpatchify: null pointer");
  SANA_REQUIRE(B > 0 && Cout > 0 && Hp > 0 && Wp > 0 && p > 0, "sana_unpatchify: sizes must be positive");
  SANA_REQUIRE(ld >= Cout * p * p, "sana_unpatchify: row stride smaller than a patch");
  SANA_REQUIRE(Hp * p < (1 << 20) && Wp * p < (1 << 20) && Cout < (1 << 20), "sana_unpatchify: size out of range");
  const int64_t total = B * Cout * Hp * p * Wp * p;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)ceil_div(total, 256);
  if (dtype == SANA_BF16)
    unpatchify_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(tok),
                                                          static_cast<__nv_bfloat16*>(out), (int)Cout, (int)Hp,
                                                          (int)Wp, (int)p, (int)ld, total);
  else if (dtype == SANA_F32)
    unpatchify_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(tok), static_cast<float*>(out), (int)Cout,
                                                  (int)Hp, (int)Wp, (int)p, (int)ld, total);
  else
    return fail(SANA_ERR_UNSUPPORTED, "sana_unpatchify: unsupported dtype %d", dtype);
  SANA_LAUNCH_CHECK("unpatchify kernel");
  return SANA_OK;
}

extern "C" int sana_timestep_embedding(const float* t, void* out, int64_t B, int64_t dim, float max_period, int dtype,
                                       void* stream) {
  SANA_REQUIRE(t && out, "sana_timestep_embedding: null pointer");
  SANA_REQUIRE(B > 0 && dim > 1 && B * dim < (1 << 30), "sana_timestep_embedding: bad sizes");
  SANA_REQUIRE(max_period > 1.0f, "sana_timestep_embedding: max_period must exceed 1");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)ceil_div(B * dim, 128);
  const float nlp = (float)(-std::log((double)max_period));
  if (dtype == SANA_BF16)
    timestep_embedding_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(t, static_cast<__nv_bfloat16*>(out), (int)B,
                                                                  (int)dim, nlp);
  else if (dtype == SANA_F32)
    timestep_embedding_kernel<float><<<grid, 128, 0, st>>>(t, static_cast<float*>(out), (int)B, (int)dim, nlp);
  else
    return fail(SANA_ERR_UNSUPPORTED, "sana_timestep_embedding: unsupported dtype %d", dtype);
  SANA_LAUNCH_CHECK("timestep_embedding kernel");
  return SANA_OK;
}

extern "C" int sana_silu(const void* x, void* out, int64_t n, int dtype, void* stream) {
  SANA_REQUIRE(x && out, "sana_silu: null pointer");
  SANA_REQUIRE(n > 0, "sana_silu: n must be positive");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)ceil_div(n, 256);
  if (dtype == SANA_BF16)
    silu_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x),
                                                    static_cast<__nv_bfloat16*>(out), n);
  else if (dtype == SANA_F32)
    silu_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), static_cast<float*>(out), n);
  else
    return fail(SANA_ERR_UNSUPPORTED, "sana_silu: unsupported dtype %d", dtype);
  SANA_LAUNCH_CHECK("silu kernel");
  return SANA_OK;
}
