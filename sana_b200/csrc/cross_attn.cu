// Softmax core of the block's cross-attention: image tokens (queries) attend to at most a few
// hundred text tokens.  out[b, n, h, :] = softmax(q k^T / sqrt(hd) + (1 - mask) * -10000) v.
//
// bf16 kernel: one CTA = 64 queries of one (batch, head), 4 warps x 16 rows.  K and V stream
// through shared memory in 64-key chunks (16-byte cp.async, double buffered, rows padded by
// 16 bytes so ldmatrix is conflict-free); S = Q K^T and O += P V run on warp-level bf16 tensor
// cores with fp32 accumulation and an online softmax in the exp2 domain; P is re-used from
// the S accumulator registers as the A operand of the second product.  Head dimensions that
// are not a multiple of 16 (72 at Sana-600M) are zero-padded in shared memory.
// fp32 kernel: one CTA per query row, plain FMA (parity path).
#include "common.cuh"

namespace sana {

constexpr int CA_BQ = 64, CA_BK = 64, CA_THREADS = 128;

__device__ __forceinline__ void ca_cp_async_16(uint32_t smem_addr, const void* gptr, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr), "l"(gptr), "r"(sz) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int HDP>
__global__ void __launch_bounds__(CA_THREADS)
cross_attn_bf16_kernel(const __nv_bfloat16* __restrict__ q, int64_t ldq, const __nv_bfloat16* __restrict__ k,
                       const __nv_bfloat16* __restrict__ v, int64_t ldkv, const __nv_bfloat16* __restrict__ mask,
                       __nv_bfloat16* __restrict__ out, int64_t ldo, int N, int L, int hd, float scale_log2e) {
  constexpr int ROW = HDP + 8;            // padded row, elements
  constexpr int ROWB = ROW * 2;           // bytes
  constexpr int KS = HDP / 16;            // k-steps of S = Q K^T
  constexpr int NT_O = HDP / 8;           // n-tiles of O
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* Qs = smem;                                   // [64][ROW]
  unsigned char* Ks = Qs + CA_BQ * ROWB;                      // [2][64][ROW]
  unsigned char* Vs = Ks + 2 * CA_BK * ROWB;                  // [2][64][ROW]
  float* bias_s = reinterpret_cast<float*>(Vs + 2 * CA_BK * ROWB);  // [nkc * 64]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int head = blockIdx.y, b = blockIdx.z;
  const int q0 = blockIdx.x * CA_BQ;
  const int nkc = (L + CA_BK - 1) / CA_BK;
  const int chunks_valid = hd >> 3, chunks_total = HDP >> 3;
  const uint32_t Qs_u = (uint32_t)__cvta_generic_to_shared(Qs);
  const uint32_t Ks_u = (uint32_t)__cvta_generic_to_shared(Ks);
  const uint32_t Vs_u = (uint32_t)__cvta_generic_to_shared(Vs);

  const __nv_bfloat16* qg = q + ((int64_t)b * N + q0) * ldq + (int64_t)head * hd;
  const __nv_bfloat16* kg = k + (int64_t)b * L * ldkv + (int64_t)head * hd;
  const __nv_bfloat16* vg = v + (int64_t)b * L * ldkv + (int64_t)head * hd;

  // zero the pad columns (dims hd .. HDP) of Q, K, V once: cp.async never writes them
  if (chunks_valid < chunks_total) {
    const int padc = chunks_total - chunks_valid;
    for (int e = tid; e < (CA_BQ + 4 * CA_BK) * padc; e += CA_THREADS) {
      const int r = e / padc, c = chunks_valid + e % padc;
      *reinterpret_cast<uint4*>(smem + r * ROWB + c * 16) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  for (int e = tid; e < nkc * CA_BK; e += CA_THREADS) {
    float bv = -INFINITY;  // keys beyond L never contribute
    if (e < L) bv = mask ? (1.0f - __bfloat162float(mask[(int64_t)b * L + e])) * (-10000.0f * 1.4426950408889634f) : 0.f;
    bias_s[e] = bv;
  }
  // Q tile and the first K/V chunk
  for (int e = tid; e < CA_BQ * chunks_valid; e += CA_THREADS) {
    const int r = e / chunks_valid, c = e % chunks_valid;
    ca_cp_async_16(Qs_u + r * ROWB + c * 16, qg + (int64_t)r * ldq + c * 8, q0 + r < N);
  }
  auto load_kv = [&](int kc, int buf) {
    for (int e = tid; e < CA_BK * chunks_valid; e += CA_THREADS) {
      const int r = e / chunks_valid, c = e % chunks_valid;
      const int key = kc * CA_BK + r;
      const bool ok = key < L;
      const int64_t off = (int64_t)(ok ? key : 0) * ldkv + c * 8;
      ca_cp_async_16(Ks_u + (buf * CA_BK + r) * ROWB + c * 16, kg + off, ok);
      ca_cp_async_16(Vs_u + (buf * CA_BK + r) * ROWB + c * 16, vg + off, ok);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  load_kv(0, 0);
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();

  // Q fragments of this warp's 16 rows stay in registers
  uint32_t qf[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    const int row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, col = ks * 16 + (lane >> 4) * 8;
    ldsm_x4(qf[ks], Qs_u + row * ROWB + col * 2);
  }
  float o[NT_O][4];
#pragma unroll
  for (int n = 0; n < NT_O; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};

  for (int kc = 0; kc < nkc; ++kc) {
    const int buf = kc & 1;
    if (kc + 1 < nkc) load_kv(kc + 1, buf ^ 1);  // the other buffer was released by the barrier below
    // ---- S = Q K^T for 64 keys
    float s[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
      for (int np = 0; np < 4; ++np) {  // two key tiles per ldmatrix.x4
        uint32_t kf[4];
        const int row = buf * CA_BK + np * 16 + (lane >> 4) * 8 + (lane & 7), col = ks * 16 + ((lane >> 3) & 1) * 8;
        ldsm_x4(kf, Ks_u + row * ROWB + col * 2);
        mma_bf16_16816(s[2 * np], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], kf[0], kf[1]);
        mma_bf16_16816(s[2 * np + 1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], kf[2], kf[3]);
      }
    }
    // ---- online softmax (exp2 domain); rows g (c0,c1) and g+8 (c2,c3)
    float mx[2] = {mrow[0], mrow[1]};
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      const float b0 = bias_s[kc * CA_BK + n * 8 + 2 * t], b1 = bias_s[kc * CA_BK + n * 8 + 2 * t + 1];
      s[n][0] = fmaf(s[n][0], scale_log2e, b0), s[n][1] = fmaf(s[n][1], scale_log2e, b1);
      s[n][2] = fmaf(s[n][2], scale_log2e, b0), s[n][3] = fmaf(s[n][3], scale_log2e, b1);
      mx[0] = fmaxf(mx[0], fmaxf(s[n][0], s[n][1]));
      mx[1] = fmaxf(mx[1], fmaxf(s[n][2], s[n][3]));
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
    float corr[2], sum[2] = {0.f, 0.f};
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      corr[r] = fast_exp2(mrow[r] - mx[r]);  // first chunk: exp2(-inf) = 0
      mrow[r] = mx[r];
    }
    uint32_t pf[4][4];  // P as A fragments: key steps of 16
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      const float p0 = fast_exp2(s[n][0] - mx[0]), p1 = fast_exp2(s[n][1] - mx[0]);
      const float p2 = fast_exp2(s[n][2] - mx[1]), p3 = fast_exp2(s[n][3] - mx[1]);
      sum[0] += p0 + p1;
      sum[1] += p2 + p3;
      pf[n >> 1][(n & 1) * 2] = pack_bf16(p0, p1);
      pf[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
      sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
      lrow[r] = lrow[r] * corr[r] + sum[r];
    }
#pragma unroll
    for (int n = 0; n < NT_O; ++n) {
      o[n][0] *= corr[0], o[n][1] *= corr[0];
      o[n][2] *= corr[1], o[n][3] *= corr[1];
    }
    // ---- O += P V
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {  // 16 keys per step
#pragma unroll
      for (int np = 0; np < NT_O / 2; ++np) {  // two dim tiles per ldmatrix.x4.trans
        uint32_t vf[4];
        const int row = buf * CA_BK + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, col = np * 16 + (lane >> 4) * 8;
        ldsm_x4_trans(vf, Vs_u + row * ROWB + col * 2);
        mma_bf16_16816(o[2 * np], pf[kk][0], pf[kk][1], pf[kk][2], pf[kk][3], vf[0], vf[1]);
        mma_bf16_16816(o[2 * np + 1], pf[kk][0], pf[kk][1], pf[kk][2], pf[kk][3], vf[2], vf[3]);
      }
    }
    if (kc + 1 < nkc) {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      __syncthreads();  // next chunk landed for everybody; everybody finished reading this one
    }
  }

  // ---- normalise, stage this warp's 16 rows in its (private) rows of the Q tile, 16-byte stores
  const float inv[2] = {1.0f / lrow[0], 1.0f / lrow[1]};
  __syncwarp();
#pragma unroll
  for (int n = 0; n < NT_O; ++n) {
    *reinterpret_cast<uint32_t*>(Qs + (warp * 16 + g) * ROWB + (n * 8 + 2 * t) * 2) = pack_bf16(o[n][0] * inv[0], o[n][1] * inv[0]);
    *reinterpret_cast<uint32_t*>(Qs + (warp * 16 + g + 8) * ROWB + (n * 8 + 2 * t) * 2) = pack_bf16(o[n][2] * inv[1], o[n][3] * inv[1]);
  }
  __syncwarp();
  __nv_bfloat16* og = out + ((int64_t)b * N + q0) * ldo + (int64_t)head * hd;
  for (int e = lane; e < 16 * chunks_valid; e += 32) {
    const int r = warp * 16 + e / chunks_valid, c = e % chunks_valid;
    if (q0 + r < N) *reinterpret_cast<uint4*>(og + (int64_t)r * ldo + c * 8) = *reinterpret_cast<const uint4*>(Qs + r * ROWB + c * 16);
  }
}

// fp32: one CTA per (query, head, batch); logits in shared memory.
__global__ void __launch_bounds__(128)
cross_attn_f32_kernel(const float* __restrict__ q, int64_t ldq, const float* __restrict__ k, const float* __restrict__ v,
                      int64_t ldkv, const float* __restrict__ mask, float* __restrict__ out, int64_t ldo, int N, int L,
                      int hd, float scale) {
  extern __shared__ float sm[];
  float* logit = sm;          // [L]
  float* qs = sm + L;         // [hd]
  __shared__ float red[4];
  const int n = blockIdx.x, head = blockIdx.y, b = blockIdx.z, tid = threadIdx.x;
  const float* qr = q + ((int64_t)b * N + n) * ldq + (int64_t)head * hd;
  for (int d = tid; d < hd; d += 128) qs[d] = qr[d];
  __syncthreads();
  float mx = -INFINITY;
  for (int j = tid; j < L; j += 128) {
    const float* kr = k + ((int64_t)b * L + j) * ldkv + (int64_t)head * hd;
    float s = 0.f;
    for (int d = 0; d < hd; ++d) s = fmaf(qs[d], kr[d], s);
    s = s * scale + (mask ? (1.0f - mask[(int64_t)b * L + j]) * -10000.0f : 0.f);
    logit[j] = s;
    mx = fmaxf(mx, s);
  }
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((tid & 31) == 0) red[tid >> 5] = mx;
  __syncthreads();
  mx = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
  __syncthreads();
  float sum = 0.f;
  for (int j = tid; j < L; j += 128) {
    const float p = expf(logit[j] - mx);
    logit[j] = p;
    sum += p;
  }
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if ((tid & 31) == 0) red[tid >> 5] = sum;
  __syncthreads();
  sum = red[0] + red[1] + red[2] + red[3];
  float* orow = out + ((int64_t)b * N + n) * ldo + (int64_t)head * hd;
  for (int d = tid; d < hd; d += 128) {
    float acc = 0.f;
    for (int j = 0; j < L; ++j) acc = fmaf(logit[j], v[((int64_t)b * L + j) * ldkv + (int64_t)head * hd + d], acc);
    orow[d] = acc / sum;
  }
}

template <int HDP>
static int launch_ca_bf16(const void* q, int64_t ldq, const void* k, const void* v, int64_t ldkv, const void* mask,
                          void* out, int64_t ldo, int64_t B, int64_t N, int64_t L, int heads, int hd, cudaStream_t st) {
  const int nkc = (int)ceil_div(L, CA_BK);
  const int smem_bytes = (CA_BQ + 4 * CA_BK) * (HDP + 8) * 2 + nkc * CA_BK * 4;
  if (smem_bytes > 227 * 1024) return fail(SANA_ERR_UNSUPPORTED, "sana_cross_attention: too many keys (%lld)", (long long)L);
  static OncePerDevice attr_once;
  if (attr_once.first_time()) {
    cudaError_t e = cudaFuncSetAttribute(cross_attn_bf16_kernel<HDP>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return cuda_status(e, "cudaFuncSetAttribute(cross_attn)");
  }
  const dim3 grid((unsigned)ceil_div(N, CA_BQ), (unsigned)heads, (unsigned)B);
  const float scale_log2e = 1.4426950408889634f / sqrtf((float)hd);
  cross_attn_bf16_kernel<HDP><<<grid, CA_THREADS, smem_bytes, st>>>(
      static_cast<const __nv_bfloat16*>(q), ldq, static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v),
      ldkv, static_cast<const __nv_bfloat16*>(mask), static_cast<__nv_bfloat16*>(out), ldo, (int)N, (int)L, hd, scale_log2e);
  SANA_LAUNCH_CHECK("cross_attn kernel");
  return SANA_OK;
}

// tensor-core kernel (cross_attn_tc.cu)
bool cross_attn_tc_supported(int64_t L, int64_t hd);
int cross_attn_tc_launch(const void* q, int64_t ldq, const void* k, const void* v, int64_t ldkv, const void* mask,
                         void* out, int64_t ldo, int64_t B, int64_t N, int64_t L, int heads, int hd, cudaStream_t st);
int cross_attn_tc_take_status(int* v);

static int g_ca_variant = 0;  // 0 = per problem, 1 = warp-level kernel, 2 = tcgen05 kernel

}  // namespace sana

using namespace sana;

extern "C" int sana_cross_attention_set_variant(int variant) {
  SANA_REQUIRE(variant >= 0 && variant <= 2, "sana_cross_attention_set_variant: variant must be 0, 1 or 2");
  g_ca_variant = variant;
  return SANA_OK;
}

extern "C" int sana_cross_attention_take_device_status(int* status_out) {
  SANA_REQUIRE(status_out, "sana_cross_attention_take_device_status: null pointer");
  return cross_attn_tc_take_status(status_out);
}

extern "C" int sana_cross_attention(const void* q, int64_t ldq, const void* k, const void* v, int64_t ldkv,
                                    const void* mask, void* out, int64_t ldo, int64_t B, int64_t N, int64_t L,
                                    int64_t heads, int64_t head_dim, int dtype, void* stream) {
  SANA_REQUIRE(q && k && v && out, "sana_cross_attention: null pointer");
  SANA_REQUIRE(B > 0 && N > 0 && L > 0 && heads > 0 && head_dim > 0, "sana_cross_attention: sizes must be positive");
  SANA_REQUIRE(B < 65536 && heads < 65536 && N < ((int64_t)1 << 30) && L < (1 << 20), "sana_cross_attention: size out of range");
  SANA_REQUIRE(head_dim % 8 == 0 && head_dim <= 128, "sana_cross_attention: head_dim must be a multiple of 8, at most 128");
  SANA_REQUIRE(ldq >= heads * head_dim && ldkv >= heads * head_dim && ldo >= heads * head_dim,
               "sana_cross_attention: row strides smaller than heads*head_dim");
  SANA_REQUIRE(ldq % 8 == 0 && ldkv % 8 == 0 && ldo % 8 == 0, "sana_cross_attention: row strides must be multiples of 8");
  SANA_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out), "sana_cross_attention: pointers must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int hd = (int)head_dim;
  if (dtype == SANA_BF16) {
    const bool tc_ok = cross_attn_tc_supported(L, head_dim);
    SANA_REQUIRE(g_ca_variant != 2 || tc_ok,
                 "sana_cross_attention: the tcgen05 kernel covers 17..304 keys and heads of 16..128 channels");
    if (tc_ok && g_ca_variant != 1)
      return cross_attn_tc_launch(q, ldq, k, v, ldkv, mask, out, ldo, B, N, L, (int)heads, hd, st);
    const int hdp = (hd + 15) / 16 * 16;
    switch (hdp) {
      case 16: case 32: return launch_ca_bf16<32>(q, ldq, k, v, ldkv, mask, out, ldo, B, N, L, (int)heads, hd, st);
      case 48: case 64: return launch_ca_bf16<64>(q, ldq, k, v, ldkv, mask, out, ldo, B, N, L, (int)heads, hd, st);
      case 80: return launch_ca_bf16<80>(q, ldq, k, v, ldkv, mask, out, ldo, B, N, L, (int)heads, hd, st);
      case 96: return launch_ca_bf16<96>(q, ldq, k, v, ldkv, mask, out, ldo, B, N, L, (int)heads, hd, st);
      case 112: return launch_ca_bf16<112>(q, ldq, k, v, ldkv, mask, out, ldo, B, N, L, (int)heads, hd, st);
      default: return launch_ca_bf16<128>(q, ldq, k, v, ldkv, mask, out, ldo, B, N, L, (int)heads, hd, st);
    }
  }
  if (dtype == SANA_F32) {
    const size_t smem_bytes = (size_t)(L + head_dim) * sizeof(float);
    SANA_REQUIRE(smem_bytes <= 48 * 1024, "sana_cross_attention (fp32): too many keys");
    SANA_REQUIRE(N < 65536 * 32768LL, "sana_cross_attention (fp32): too many queries");
    const dim3 grid((unsigned)N, (unsigned)heads, (unsigned)B);
    cross_attn_f32_kernel<<<grid, 128, smem_bytes, st>>>(static_cast<const float*>(q), ldq, static_cast<const float*>(k),
                                                         static_cast<const float*>(v), ldkv, static_cast<const float*>(mask),
                                                         static_cast<float*>(out), ldo, (int)N, (int)L, hd,
                                                         1.0f / sqrtf((float)hd));
    SANA_LAUNCH_CHECK("cross_attn (fp32) kernel");
    return SANA_OK;
  }
  return fail(SANA_ERR_UNSUPPORTED, "sana_cross_attention: unsupported dtype %d", dtype);
}
