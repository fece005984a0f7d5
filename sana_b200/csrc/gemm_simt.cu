// SIMT projection kernel: out = epilogue(A @ Wt^T) with fp32 FMA accumulation.
// Product path for fp32 tensors (the fp32 parity configuration); for bf16 it is only a
// device-side cross-check of the tensor-core kernel.
#include "epilogue.cuh"

namespace sana {

constexpr int SG_BM = 64, SG_BN = 64, SG_BK = 16;

template <typename T>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const T* __restrict__ A, int64_t lda, const T* __restrict__ W, int64_t ldw, T* __restrict__ out,
                 int64_t ldo, int64_t M, int64_t N, int64_t K, const EpiParams ep) {
  __shared__ float As[SG_BK][SG_BM + 4];
  __shared__ float Ws[SG_BK][SG_BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, 4 x 4 outputs each
  const int64_t m0 = (int64_t)blockIdx.y * SG_BM, n0 = (int64_t)blockIdx.x * SG_BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int64_t k0 = 0; k0 < K; k0 += SG_BK) {
    for (int e = tid; e < SG_BM * SG_BK; e += 256) {
      const int r = e / SG_BK, c = e % SG_BK;
      const int64_t m = m0 + r, k = k0 + c;
      As[c][r] = (m < M && k < K) ? to_f32(A[m * lda + k]) : 0.f;
      const int64_t n = n0 + r;
      Ws[c][r] = (n < N && k < K) ? to_f32(W[n * ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < SG_BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t n = n0 + tx * 4 + j;
      if (n < N) out[m * ldo + n] = from_f32<T>(epi_scalar<T>(acc[i][j], m, n, N, ep));
    }
  }
}

int gemm_simt_launch(const void* A, int64_t lda, const void* Wt, int64_t ldw, void* out, int64_t ldo, int64_t M,
                     int64_t N, int64_t K, const EpiParams& ep, int dtype, cudaStream_t st) {
  const dim3 grid((unsigned)ceil_div(N, SG_BN), (unsigned)ceil_div(M, SG_BM));
  if (grid.y >= 65536) return fail(SANA_ERR_INVALID, "sana_gemm (simt): M too large");
  if (dtype == SANA_F32) {
    gemm_simt_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(A), lda, static_cast<const float*>(Wt),
                                                  ldw, static_cast<float*>(out), ldo, M, N, K, ep);
  } else if (dtype == SANA_BF16) {
    gemm_simt_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(A), lda,
                                                          static_cast<const __nv_bfloat16*>(Wt), ldw,
                                                          static_cast<__nv_bfloat16*>(out), ldo, M, N, K, ep);
  } else {
    return fail(SANA_ERR_UNSUPPORTED, "sana_gemm: unsupported dtype %d", dtype);
  }
  SANA_LAUNCH_CHECK("gemm_simt kernel");
  return SANA_OK;
}

}  // namespace sana

using namespace sana;

static int check_gemm_args(const char* who, const void* A, int64_t lda, const void* Wt, int64_t ldw, void* out,
                           int64_t ldo, int64_t M, int64_t N, int64_t K) {
  SANA_REQUIRE(A && Wt && out, "%s: null pointer", who);
  SANA_REQUIRE(M > 0 && N > 0 && K > 0, "%s: M, N, K must be positive", who);
  SANA_REQUIRE(lda >= K && ldw >= K && ldo >= N, "%s: row stride smaller than the row", who);
  SANA_REQUIRE(M < ((int64_t)1 << 31) && N < ((int64_t)1 << 31) && K < ((int64_t)1 << 31), "%s: size out of range", who);
  return SANA_OK;
}

extern "C" int sana_gemm_simt(const void* A, int64_t lda, const void* Wt, int64_t ldw, void* out, int64_t ldo,
                              int64_t M, int64_t N, int64_t K, const sana_gemm_epilogue* ep, int dtype, void* stream) {
  int rc = check_gemm_args("sana_gemm_simt", A, lda, Wt, ldw, out, ldo, M, N, K);
  if (rc) return rc;
  EpiParams p;
  rc = check_epilogue(ep, N, &p, "sana_gemm_simt");
  if (rc) return rc;
  return gemm_simt_launch(A, lda, Wt, ldw, out, ldo, M, N, K, p, dtype, static_cast<cudaStream_t>(stream));
}

namespace sana {
int gemm_tc_launch(const void* A, int64_t lda, const void* Wt, int64_t ldw, void* out, int64_t ldo, int64_t M,
                   int64_t N, int64_t K, const EpiParams& ep, cudaStream_t st);
}

extern "C" int sana_gemm(const void* A, int64_t lda, const void* Wt, int64_t ldw, void* out, int64_t ldo, int64_t M,
                         int64_t N, int64_t K, const sana_gemm_epilogue* ep, int dtype, void* stream) {
  int rc = check_gemm_args("sana_gemm", A, lda, Wt, ldw, out, ldo, M, N, K);
  if (rc) return rc;
  EpiParams p;
  rc = check_epilogue(ep, N, &p, "sana_gemm");
  if (rc) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == SANA_BF16) return gemm_tc_launch(A, lda, Wt, ldw, out, ldo, M, N, K, p, st);
  if (dtype == SANA_F32) return gemm_simt_launch(A, lda, Wt, ldw, out, ldo, M, N, K, p, dtype, st);
  return fail(SANA_ERR_UNSUPPORTED, "sana_gemm: unsupported dtype %d", dtype);
}
