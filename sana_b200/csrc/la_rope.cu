// ReLU linear attention with a rotation of the numerator's q and k (the self-attention of
// Sana-Video): per-head (D+1) x D state reduction and apply + normalise, for heads of D channels,
// D a multiple of 16 up to 128.
//
//   state[i][j] = sum_n v[n][i] * rot(relu(k[n]))[j]   (i < D),   state[D][j] = sum_n relu(k[n][j])
//   out[n][i]   = (sum_j state[i][j] * rot(relu(q[n]))[j]) / (sum_j state[D][j] * relu(q[n][j]) + eps)
//   rot(x)[2p] = x[2p] cos[n][p] - x[2p+1] sin[n][p],  rot(x)[2p+1] = x[2p] sin[n][p] + x[2p+1] cos[n][p]
//
// bf16: one CTA per (head, token chunk, sample).  A tile of 64 tokens is loaded 16 bytes per
// lane, passed through ReLU and the rotation once, and written to shared memory as bf16; the
// products run on warp-level bf16 tensor-core instructions with fp32 accumulation, fed by
// ldmatrix from rows padded by 16 bytes (conflict-free).  The key sum and the normaliser stay
// in fp32 on the CUDA cores.  fp32: plain FFMA kernels (the parity path).
#include "common.cuh"
#include "la_plan.cuh"

namespace sana {

constexpr int LR_THREADS = 256;
constexpr int LR_TOK = 64;   // tokens per tile, bf16 kernels
constexpr int LR_TOKF = 16;  // tokens per tile, fp32 kernels

__device__ __forceinline__ void lr_ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void lr_ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// ReLU of 8 bf16 channels (4 rotation pairs) of one token: x = relu(raw) in fp32, and
// rot = the rotated pairs packed back to bf16.
__device__ __forceinline__ void lr_relu_rotate8(const uint4 raw, const float4 c, const float4 s, float (&x)[8],
                                                uint4* rot) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  const float cc[4] = {c.x, c.y, c.z, c.w}, ss[4] = {s.x, s.y, s.z, s.w};
  uint32_t o[4];
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const float x0 = fmaxf(bf16_lo(w[p]), 0.f), x1 = fmaxf(bf16_hi(w[p]), 0.f);
    x[2 * p] = x0, x[2 * p + 1] = x1;
    o[p] = pack_bf16(x0 * cc[p] - x1 * ss[p], x0 * ss[p] + x1 * cc[p]);
  }
  *rot = make_uint4(o[0], o[1], o[2], o[3]);
}

// ------------------------------------------------------------------------------------------
// state, bf16.  grid (H, chunks, B) - heads fastest, so that CTAs running at the same time read
// whole token rows between them.  Staging: 16 lanes per token (lane group `grp` owns channels
// 8 grp .. 8 grp + 7 and keeps their key sum in registers), 16 tokens per pass, 4 passes per tile;
// two CTAs per SM, so that one stages while the other multiplies.
// Products: warp w < D/16 owns value channels 16 w .. 16 w + 15 (one M tile) against all D key
// channels; tokens are the contraction index, so both operands are read with ldmatrix.trans from
// the token-major tiles.
// ------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(LR_THREADS, 2)
la_rope_state_bf16_kernel(const __nv_bfloat16* __restrict__ kp, const __nv_bfloat16* __restrict__ vp, int64_t ld,
                          const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                          float* __restrict__ partial, int N, int H, int Lc, int nchunks) {
  constexpr int G = D / 8;        // 16-byte groups per token row
  constexpr int ROW = D + 8;      // padded row, elements
  constexpr int ROWB = ROW * 2;   // bytes
  constexpr int MT = D / 16;      // M tiles = warps that multiply
  constexpr int NP = D / 16;      // pairs of N tiles
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* Ks = smem;                   // [64][ROW] rotated relu(k)
  unsigned char* Vs = smem + LR_TOK * ROWB;   // [64][ROW] v
  const uint32_t Ks_u = (uint32_t)__cvta_generic_to_shared(Ks);
  const uint32_t Vs_u = (uint32_t)__cvta_generic_to_shared(Vs);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int slot = tid >> 4, grp = tid & 15;
  const int h = blockIdx.x, chunk = blockIdx.y, b = blockIdx.z;
  const int n_begin = chunk * Lc, n_end = min(N, n_begin + Lc);
  const bool loader = grp < G;
  const int64_t col = (int64_t)h * D + 8 * grp;
  const __nv_bfloat16* kbase = kp + (int64_t)b * N * ld + col;
  const __nv_bfloat16* vbase = vp + (int64_t)b * N * ld + col;

  float ksum[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) ksum[e] = 0.f;
  float acc[2 * NP][4];
#pragma unroll
  for (int n = 0; n < 2 * NP; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;

  for (int n0 = n_begin; n0 < n_end; n0 += LR_TOK) {
    if (loader) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {  // two passes at a time keep the staging registers low
        uint4 kr[2], vr[2];
        float4 cr[2], sr[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int tok = n0 + 16 * (2 * half + r) + slot;
          if (tok < n_end) {
            kr[r] = ldg_nc_u4(kbase + (int64_t)tok * ld);
            vr[r] = ldg_nc_u4(vbase + (int64_t)tok * ld);
            cr[r] = __ldg(reinterpret_cast<const float4*>(cos_t + (int64_t)tok * (D / 2) + 4 * grp));
            sr[r] = __ldg(reinterpret_cast<const float4*>(sin_t + (int64_t)tok * (D / 2) + 4 * grp));
          } else {
            kr[r] = vr[r] = make_uint4(0u, 0u, 0u, 0u);
            cr[r] = sr[r] = make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          float x[8];
          uint4 rot;
          lr_relu_rotate8(kr[r], cr[r], sr[r], x, &rot);
#pragma unroll
          for (int e = 0; e < 8; ++e) ksum[e] += x[e];
          const int row = 16 * (2 * half + r) + slot;
          *reinterpret_cast<uint4*>(Ks + row * ROWB + grp * 16) = rot;
          *reinterpret_cast<uint4*>(Vs + row * ROWB + grp * 16) = vr[r];
        }
      }
    }
    __syncthreads();
    if (warp < MT) {
#pragma unroll
      for (int ks = 0; ks < LR_TOK / 16; ++ks) {
        uint32_t af[4];
        {
          const int row = ks * 16 + (lane & 7) + (lane >> 4) * 8, ch = warp * 16 + ((lane >> 3) & 1) * 8;
          lr_ldsm_x4_trans(af, Vs_u + row * ROWB + ch * 2);
        }
#pragma unroll
        for (int np = 0; np < NP; ++np) {
          uint32_t bf[4];
          const int row = ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, ch = np * 16 + (lane >> 4) * 8;
          lr_ldsm_x4_trans(bf, Ks_u + row * ROWB + ch * 2);
          mma_bf16_16816(acc[2 * np], af[0], af[1], af[2], af[3], bf[0], bf[1]);
          mma_bf16_16816(acc[2 * np + 1], af[0], af[1], af[2], af[3], bf[2], bf[3]);
        }
      }
    }
    __syncthreads();
  }

  float* out = partial + (((int64_t)b * nchunks + chunk) * H + h) * (int64_t)((D + 1) * D);
  if (warp < MT) {
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int nt = 0; nt < 2 * NP; ++nt) {
      const int i = warp * 16 + g, j = nt * 8 + 2 * t;
      *reinterpret_cast<float2*>(out + i * D + j) = make_float2(acc[nt][0], acc[nt][1]);
      *reinterpret_cast<float2*>(out + (i + 8) * D + j) = make_float2(acc[nt][2], acc[nt][3]);
    }
  }
  // key sum: the 16 token slots add in a fixed order
  float* red = reinterpret_cast<float*>(smem);  // [16][D]; the tiles are no longer read
  if (loader) {
#pragma unroll
    for (int e = 0; e < 8; ++e) red[slot * D + 8 * grp + e] = ksum[e];
  }
  __syncthreads();
  if (tid < D) {
    float s = 0.f;
#pragma unroll
    for (int r = 0; r < 16; ++r) s += red[r * D + tid];
    out[D * D + tid] = s;
  }
}

// ------------------------------------------------------------------------------------------
// apply, bf16.  grid (H, chunks, B).  The head's state is converted once to bf16 in shared memory
// ([i][j], j contiguous = the "col" B operand), the key-sum row stays fp32.  Staging as in the
// state kernel; the 16 lanes of a token also reduce its normaliser with shuffles.  Products:
// warp w owns tokens 16 (w & 3) .. + 15 of the tile and the value channels of half (w >> 2).
// The results go back through the token tile so that global stores are 16 bytes per lane.
// ------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(LR_THREADS)
la_rope_apply_bf16_kernel(const __nv_bfloat16* __restrict__ qp, int64_t ldq, const float* __restrict__ cos_t,
                          const float* __restrict__ sin_t, const float* __restrict__ state,
                          __nv_bfloat16* __restrict__ op, int64_t ldo, int N, int H, int Lc, float eps) {
  constexpr int G = D / 8;
  constexpr int ROW = D + 8;
  constexpr int ROWB = ROW * 2;
  constexpr int KS = D / 16;       // k-steps over the key channels
  constexpr int NTW = D / 16;      // N tiles (value channels / 8) per warp: half of D / 8
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* Ss = smem;                                  // [D + 8][ROW] bf16 state, 8 spare rows
  unsigned char* Qs = Ss + (D + 8) * ROWB;                   // [64][ROW] rotated relu(q), then the results
  float* ksum_s = reinterpret_cast<float*>(Qs + LR_TOK * ROWB);  // [D]
  float* rden_s = ksum_s + D;                                // [64] 1 / (normaliser + eps)
  const uint32_t Ss_u = (uint32_t)__cvta_generic_to_shared(Ss);
  const uint32_t Qs_u = (uint32_t)__cvta_generic_to_shared(Qs);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int slot = tid >> 4, grp = tid & 15;
  const int h = blockIdx.x, chunk = blockIdx.y, b = blockIdx.z;
  const int n_begin = chunk * Lc, n_end = min(N, n_begin + Lc);
  const bool loader = grp < G;

  const float* sg = state + ((int64_t)b * H + h) * (int64_t)((D + 1) * D);
  for (int e = tid; e < D * (D / 2); e += LR_THREADS) {
    const int i = e / (D / 2), jp = e % (D / 2);
    const float2 s2 = __ldg(reinterpret_cast<const float2*>(sg + i * D + 2 * jp));
    *reinterpret_cast<uint32_t*>(Ss + i * ROWB + jp * 4) = pack_bf16(s2.x, s2.y);
  }
  for (int e = tid; e < 8 * (ROW / 2); e += LR_THREADS)  // spare rows: read by the last odd tile, never used
    *reinterpret_cast<uint32_t*>(Ss + D * ROWB + e * 4) = 0u;
  if (tid < D) ksum_s[tid] = __ldg(sg + D * D + tid);
  __syncthreads();

  float kreg[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) kreg[e] = loader ? ksum_s[8 * grp + e] : 0.f;
  const int64_t col = (int64_t)h * D + 8 * grp;
  const __nv_bfloat16* qbase = qp + (int64_t)b * N * ldq + col;
  __nv_bfloat16* obase = op + (int64_t)b * N * ldo + col;
  const int mtile = warp & 3, nhalf = warp >> 2;

  for (int n0 = n_begin; n0 < n_end; n0 += LR_TOK) {
    {
      uint4 qr[4];
      float4 cr[4], sr[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int tok = n0 + 16 * r + slot;
        if (loader && tok < n_end) {
          qr[r] = ldg_nc_u4(qbase + (int64_t)tok * ldq);
          cr[r] = __ldg(reinterpret_cast<const float4*>(cos_t + (int64_t)tok * (D / 2) + 4 * grp));
          sr[r] = __ldg(reinterpret_cast<const float4*>(sin_t + (int64_t)tok * (D / 2) + 4 * grp));
        } else {
          qr[r] = make_uint4(0u, 0u, 0u, 0u);
          cr[r] = sr[r] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        float x[8];
        uint4 rot;
        lr_relu_rotate8(qr[r], cr[r], sr[r], x, &rot);
        float den = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) den = fmaf(x[e], kreg[e], den);
        // all 32 lanes take part: the 16 lanes of a token are one half of a warp
        den += __shfl_xor_sync(0xffffffffu, den, 1);
        den += __shfl_xor_sync(0xffffffffu, den, 2);
        den += __shfl_xor_sync(0xffffffffu, den, 4);
        den += __shfl_xor_sync(0xffffffffu, den, 8);
        const int row = 16 * r + slot;
        if (grp == 0) rden_s[row] = 1.0f / (den + eps);
        if (loader) *reinterpret_cast<uint4*>(Qs + row * ROWB + grp * 16) = rot;
      }
    }
    __syncthreads();
    float acc[NTW][4];
#pragma unroll
    for (int n = 0; n < NTW; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      uint32_t af[4];
      {
        const int row = mtile * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, ch = ks * 16 + (lane >> 4) * 8;
        lr_ldsm_x4(af, Qs_u + row * ROWB + ch * 2);
      }
#pragma unroll
      for (int np = 0; np < (NTW + 1) / 2; ++np) {
        uint32_t bf[4];
        // value channels 8 (nhalf NTW + 2 np) .. + 15; beyond D only the spare rows are touched
        const int row = (nhalf * NTW + 2 * np) * 8 + (lane >> 4) * 8 + (lane & 7), ch = ks * 16 + ((lane >> 3) & 1) * 8;
        lr_ldsm_x4(bf, Ss_u + row * ROWB + ch * 2);
        mma_bf16_16816(acc[2 * np], af[0], af[1], af[2], af[3], bf[0], bf[1]);
        if (2 * np + 1 < NTW) mma_bf16_16816(acc[2 * np + 1], af[0], af[1], af[2], af[3], bf[2], bf[3]);
      }
    }
    __syncthreads();  // every warp has read its q fragments: the tile can take the results
    {
      const int g = lane >> 2, t = lane & 3;
      const int r0 = mtile * 16 + g;
      const float d0 = rden_s[r0], d1 = rden_s[r0 + 8];
#pragma unroll
      for (int nt = 0; nt < NTW; ++nt) {
        const int i = (nhalf * NTW + nt) * 8 + 2 * t;
        *reinterpret_cast<uint32_t*>(Qs + r0 * ROWB + i * 2) = pack_bf16(acc[nt][0] * d0, acc[nt][1] * d0);
        *reinterpret_cast<uint32_t*>(Qs + (r0 + 8) * ROWB + i * 2) = pack_bf16(acc[nt][2] * d1, acc[nt][3] * d1);
      }
    }
    __syncthreads();
    if (loader) {
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int tok = n0 + 16 * r + slot, row = 16 * r + slot;
        if (tok < n_end)
          *reinterpret_cast<uint4*>(obase + (int64_t)tok * ldo) = *reinterpret_cast<const uint4*>(Qs + row * ROWB + grp * 16);
      }
    }
    // the next tile's staging writes exactly the elements this thread has just read
  }
}

// ------------------------------------------------------------------------------------------
// fp32 kernels (FFMA).  state: grid (chunks, H, B); thread (ti = tid >> 4, tj = tid & 15) owns
// state[ti + 16 a][tj + 16 b], a, b < D / 16; threads tid < D also own the key sum of channel tid.
// ------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(LR_THREADS)
la_rope_state_f32_kernel(const float* __restrict__ kp, const float* __restrict__ vp, int64_t ld,
                         const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                         float* __restrict__ partial, int N, int H, int Lc, int nchunks) {
  constexpr int T = D / 16;
  __shared__ float kr[LR_TOKF][D], kw[LR_TOKF][D], vs[LR_TOKF][D];
  const int tid = threadIdx.x, ti = tid >> 4, tj = tid & 15;
  const int chunk = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int n_begin = chunk * Lc, n_end = min(N, n_begin + Lc);
  const float* kbase = kp + (int64_t)b * N * ld + (int64_t)h * D;
  const float* vbase = vp + (int64_t)b * N * ld + (int64_t)h * D;
  float acc[T][T];
#pragma unroll
  for (int a = 0; a < T; ++a)
#pragma unroll
    for (int c = 0; c < T; ++c) acc[a][c] = 0.f;
  float ks = 0.f;
  for (int n0 = n_begin; n0 < n_end; n0 += LR_TOKF) {
    for (int e = tid; e < LR_TOKF * (D / 2); e += LR_THREADS) {
      const int r = e / (D / 2), p = e % (D / 2), tok = n0 + r;
      float2 k2 = make_float2(0.f, 0.f), v2 = k2;
      float c = 0.f, s = 0.f;
      if (tok < n_end) {
        k2 = *reinterpret_cast<const float2*>(kbase + (int64_t)tok * ld + 2 * p);
        v2 = *reinterpret_cast<const float2*>(vbase + (int64_t)tok * ld + 2 * p);
        c = cos_t[(int64_t)tok * (D / 2) + p], s = sin_t[(int64_t)tok * (D / 2) + p];
      }
      const float x0 = fmaxf(k2.x, 0.f), x1 = fmaxf(k2.y, 0.f);
      kw[r][2 * p] = x0, kw[r][2 * p + 1] = x1;
      kr[r][2 * p] = x0 * c - x1 * s, kr[r][2 * p + 1] = x0 * s + x1 * c;
      vs[r][2 * p] = v2.x, vs[r][2 * p + 1] = v2.y;
    }
    __syncthreads();
#pragma unroll 4
    for (int r = 0; r < LR_TOKF; ++r) {
      float vi[T], kj[T];
#pragma unroll
      for (int a = 0; a < T; ++a) vi[a] = vs[r][ti + 16 * a], kj[a] = kr[r][tj + 16 * a];
#pragma unroll
      for (int a = 0; a < T; ++a)
#pragma unroll
        for (int c = 0; c < T; ++c) acc[a][c] = fmaf(vi[a], kj[c], acc[a][c]);
    }
    if (tid < D) {
#pragma unroll
      for (int r = 0; r < LR_TOKF; ++r) ks += kw[r][tid];
    }
    __syncthreads();
  }
  float* out = partial + (((int64_t)b * nchunks + chunk) * H + h) * (int64_t)((D + 1) * D);
#pragma unroll
  for (int a = 0; a < T; ++a)
#pragma unroll
    for (int c = 0; c < T; ++c) out[(ti + 16 * a) * D + tj + 16 * c] = acc[a][c];
  if (tid < D) out[D * D + tid] = ks;
}

// apply, fp32.  grid (chunks, H, B); the state sits in shared memory with rows padded to D + 1
// floats; thread (tn = tid >> 4, ti = tid & 15) owns token tn of a 16-token tile and value
// channels ti + 16 a.
template <int D>
__global__ void __launch_bounds__(LR_THREADS)
la_rope_apply_f32_kernel(const float* __restrict__ qp, int64_t ldq, const float* __restrict__ cos_t,
                         const float* __restrict__ sin_t, const float* __restrict__ state, float* __restrict__ op,
                         int64_t ldo, int N, int H, int Lc, float eps) {
  constexpr int T = D / 16;
  extern __shared__ __align__(16) float fsm[];
  float* Sf = fsm;                      // [D][D + 1]
  float* ksum_s = Sf + D * (D + 1);     // [D]
  float* qr = ksum_s + D;               // [16][D] rotated
  float* qw = qr + LR_TOKF * D;         // [16][D] relu only
  const int tid = threadIdx.x, tn = tid >> 4, ti = tid & 15;
  const int chunk = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int n_begin = chunk * Lc, n_end = min(N, n_begin + Lc);
  const float* sg = state + ((int64_t)b * H + h) * (int64_t)((D + 1) * D);
  for (int e = tid; e < D * D; e += LR_THREADS) Sf[(e / D) * (D + 1) + e % D] = sg[e];
  if (tid < D) ksum_s[tid] = sg[D * D + tid];
  const float* qbase = qp + (int64_t)b * N * ldq + (int64_t)h * D;
  float* obase = op + (int64_t)b * N * ldo + (int64_t)h * D;
  for (int n0 = n_begin; n0 < n_end; n0 += LR_TOKF) {
    __syncthreads();  // state loaded / previous tile consumed
    for (int e = tid; e < LR_TOKF * (D / 2); e += LR_THREADS) {
      const int r = e / (D / 2), p = e % (D / 2), tok = n0 + r;
      float2 q2 = make_float2(0.f, 0.f);
      float c = 0.f, s = 0.f;
      if (tok < n_end) {
        q2 = *reinterpret_cast<const float2*>(qbase + (int64_t)tok * ldq + 2 * p);
        c = cos_t[(int64_t)tok * (D / 2) + p], s = sin_t[(int64_t)tok * (D / 2) + p];
      }
      const float x0 = fmaxf(q2.x, 0.f), x1 = fmaxf(q2.y, 0.f);
      qw[r * D + 2 * p] = x0, qw[r * D + 2 * p + 1] = x1;
      qr[r * D + 2 * p] = x0 * c - x1 * s, qr[r * D + 2 * p + 1] = x0 * s + x1 * c;
    }
    __syncthreads();
    float acc[T], den = 0.f;
#pragma unroll
    for (int a = 0; a < T; ++a) acc[a] = 0.f;
    for (int j = 0; j < D; ++j) {
      const float qv = qr[tn * D + j];
      den = fmaf(ksum_s[j], qw[tn * D + j], den);
#pragma unroll
      for (int a = 0; a < T; ++a) acc[a] = fmaf(Sf[(ti + 16 * a) * (D + 1) + j], qv, acc[a]);
    }
    const int tok = n0 + tn;
    if (tok < n_end) {
      const float rd = 1.0f / (den + eps);
#pragma unroll
      for (int a = 0; a < T; ++a) obase[(int64_t)tok * ldo + ti + 16 * a] = acc[a] * rd;
    }
  }
}

// Adds the per-chunk partial states in chunk order (fixed order => bit-reproducible).
__global__ void la_rope_reduce_kernel(const float* __restrict__ partial, float* __restrict__ state, int nchunks,
                                      int64_t per_batch, int64_t total) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int64_t b = idx / per_batch, r = idx - b * per_batch;
  const float* p = partial + b * nchunks * per_batch + r;
  float s = 0.f;
  for (int c = 0; c < nchunks; ++c) s += p[(int64_t)c * per_batch];
  state[idx] = s;
}

// ---- host side -------------------------------------------------------------------------------
template <int D>
struct LrSizes {
  static constexpr size_t state_bf16 = 2 * LR_TOK * (D + 8) * 2;  // also >= 16 * D floats of the final key-sum pass
  static constexpr size_t apply_bf16 = (size_t)(D + 8) * (D + 8) * 2 + LR_TOK * (D + 8) * 2 + (D + LR_TOK) * 4;
  static constexpr size_t apply_f32 = ((size_t)D * (D + 1) + D + 2 * LR_TOKF * D) * 4;
};
static_assert(LrSizes<16>::state_bf16 >= 16 * 16 * 4 && LrSizes<128>::state_bf16 >= 16 * 128 * 4, "key-sum scratch");

template <int D>
static int lr_prepare() {
  static OncePerDevice once;
  if (!once.first_time()) return SANA_OK;
  cudaError_t e = cudaFuncSetAttribute(la_rope_apply_bf16_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)LrSizes<D>::apply_bf16);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(la_rope_apply_f32_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)LrSizes<D>::apply_f32);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(la_rope_state_bf16_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)LrSizes<D>::state_bf16);
  return cuda_status(e, "la_rope: cudaFuncSetAttribute");
}

// Chunking of the token axis.  Does not depend on dtype, so that the workspace query needs none.
template <int D>
static void lr_state_plan(int64_t B, int64_t N, int64_t H, int* Lc, int* nchunks) {
  static const int64_t per_sm = resident_ctas(la_rope_state_bf16_kernel<D>, LR_THREADS, LrSizes<D>::state_bf16) / sm_count();
  // a chunk's partial state ((D+1) x D fp32, written and re-read) costs as much as ~2 D tokens of k + v
  la_chunking(B * H, N, per_sm * sm_count(), 2 * D, Lc, nchunks);
}

template <int D>
static int lr_state(const void* k, const void* v, int64_t ld, const float* cos_t, const float* sin_t, float* state,
                    float* partial, int64_t B, int64_t N, int64_t H, int dtype, cudaStream_t st) {
  int rc = lr_prepare<D>();
  if (rc != SANA_OK) return rc;
  int Lc, nchunks;
  lr_state_plan<D>(B, N, H, &Lc, &nchunks);
  if (dtype == SANA_BF16) {
    dim3 grid((unsigned)H, nchunks, (unsigned)B);
    la_rope_state_bf16_kernel<D><<<grid, LR_THREADS, LrSizes<D>::state_bf16, st>>>(
        static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), ld, cos_t, sin_t, partial, (int)N,
        (int)H, Lc, nchunks);
  } else {
    dim3 grid(nchunks, (unsigned)H, (unsigned)B);
    la_rope_state_f32_kernel<D><<<grid, LR_THREADS, 0, st>>>(static_cast<const float*>(k), static_cast<const float*>(v),
                                                           ld, cos_t, sin_t, partial, (int)N, (int)H, Lc, nchunks);
  }
  SANA_LAUNCH_CHECK("la_rope_state kernel");
  const int64_t per_batch = H * (int64_t)((D + 1) * D), total = B * per_batch;
  la_rope_reduce_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, st>>>(partial, state, nchunks, per_batch, total);
  SANA_LAUNCH_CHECK("la_rope_reduce kernel");
  return SANA_OK;
}

template <int D>
static int lr_apply(const void* q, int64_t ldq, const float* cos_t, const float* sin_t, const float* state, void* out,
                    int64_t ldo, int64_t B, int64_t N, int64_t H, float eps, int dtype, cudaStream_t st) {
  int rc = lr_prepare<D>();
  if (rc != SANA_OK) return rc;
  int Lc, nchunks;
  if (dtype == SANA_BF16) {
    static const int64_t per_sm =
        resident_ctas(la_rope_apply_bf16_kernel<D>, LR_THREADS, LrSizes<D>::apply_bf16) / sm_count();
    // loading the head's state costs about as much as D / 2 tokens of q + out
    la_chunking(B * H, N, per_sm * sm_count(), D / 2, &Lc, &nchunks);
    dim3 grid((unsigned)H, nchunks, (unsigned)B);
    la_rope_apply_bf16_kernel<D><<<grid, LR_THREADS, LrSizes<D>::apply_bf16, st>>>(
        static_cast<const __nv_bfloat16*>(q), ldq, cos_t, sin_t, state, static_cast<__nv_bfloat16*>(out), ldo, (int)N,
        (int)H, Lc, eps);
  } else {
    la_chunking(B * H, N, (int64_t)sm_count() * 2, D / 2, &Lc, &nchunks);
    dim3 grid(nchunks, (unsigned)H, (unsigned)B);
    la_rope_apply_f32_kernel<D><<<grid, LR_THREADS, LrSizes<D>::apply_f32, st>>>(
        static_cast<const float*>(q), ldq, cos_t, sin_t, state, static_cast<float*>(out), ldo, (int)N, (int)H, Lc, eps);
  }
  SANA_LAUNCH_CHECK("la_rope_apply kernel");
  return SANA_OK;
}

#define LR_DISPATCH(D, CALL)        \
  switch (D) {                      \
    case 16: return CALL(16);       \
    case 32: return CALL(32);       \
    case 48: return CALL(48);       \
    case 64: return CALL(64);       \
    case 80: return CALL(80);       \
    case 96: return CALL(96);       \
    case 112: return CALL(112);     \
    case 128: return CALL(128);     \
    default: break;                 \
  }

static int64_t lr_workspace_bytes(int64_t B, int64_t N, int64_t H, int64_t D) {
  int Lc = 0, nchunks = 0;
#define LR_PLAN(DD)                               \
  (lr_state_plan<DD>(B, N, H, &Lc, &nchunks), 0)
  switch (D) {
    case 16: LR_PLAN(16); break;
    case 32: LR_PLAN(32); break;
    case 48: LR_PLAN(48); break;
    case 64: LR_PLAN(64); break;
    case 80: LR_PLAN(80); break;
    case 96: LR_PLAN(96); break;
    case 112: LR_PLAN(112); break;
    case 128: LR_PLAN(128); break;
    default: return 0;
  }
#undef LR_PLAN
  return B * (int64_t)nchunks * H * (D + 1) * D * (int64_t)sizeof(float);
}

static bool lr_head_dim_ok(int64_t D) { return D >= 16 && D <= 128 && D % 16 == 0; }

}  // namespace sana

using namespace sana;

extern "C" int64_t sana_la_rope_state_workspace_bytes(int64_t B, int64_t N, int64_t H, int64_t D) {
  if (B <= 0 || N <= 0 || H <= 0 || !lr_head_dim_ok(D)) return 0;
  return lr_workspace_bytes(B, N, H, D);
}

extern "C" int sana_la_rope_state(const void* k, const void* v, int64_t ld, const float* cos_table,
                                  const float* sin_table, float* state, void* workspace, int64_t workspace_bytes,
                                  int64_t B, int64_t N, int64_t H, int64_t D, int dtype, void* stream) {
  SANA_REQUIRE(k && v && cos_table && sin_table && state && workspace, "sana_la_rope_state: null pointer");
  SANA_REQUIRE(B > 0 && N > 0 && H > 0, "sana_la_rope_state: B, N, H must be positive");
  SANA_REQUIRE(lr_head_dim_ok(D), "sana_la_rope_state: head dimension must be a multiple of 16 in [16, 128]");
  SANA_REQUIRE(N < (1 << 30) && B < 65536 && H < 65536, "sana_la_rope_state: size out of range");
  SANA_REQUIRE(dtype == SANA_BF16 || dtype == SANA_F32, "sana_la_rope_state: unsupported dtype");
  SANA_REQUIRE(ld >= H * D && ld % 8 == 0, "sana_la_rope_state: ld must be >= H*D and a multiple of 8");
  SANA_REQUIRE(aligned16(k) && aligned16(v) && aligned16(cos_table) && aligned16(sin_table) && aligned16(state) &&
                   aligned16(workspace),
               "sana_la_rope_state: pointers must be 16-byte aligned");
  SANA_REQUIRE(workspace_bytes >= lr_workspace_bytes(B, N, H, D), "sana_la_rope_state: workspace too small");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* partial = static_cast<float*>(workspace);
#define LR_STATE(DD) lr_state<DD>(k, v, ld, cos_table, sin_table, state, partial, B, N, H, dtype, st)
  LR_DISPATCH(D, LR_STATE)
#undef LR_STATE
  return fail(SANA_ERR_INVALID, "sana_la_rope_state: head dimension %lld", (long long)D);
}

extern "C" int sana_la_rope_apply(const void* q, int64_t ldq, const float* cos_table, const float* sin_table,
                                  const float* state, void* out, int64_t ldo, int64_t B, int64_t N, int64_t H,
                                  int64_t D, float eps, int dtype, void* stream) {
  SANA_REQUIRE(q && cos_table && sin_table && state && out, "sana_la_rope_apply: null pointer");
  SANA_REQUIRE(B > 0 && N > 0 && H > 0, "sana_la_rope_apply: B, N, H must be positive");
  SANA_REQUIRE(lr_head_dim_ok(D), "sana_la_rope_apply: head dimension must be a multiple of 16 in [16, 128]");
  SANA_REQUIRE(N < (1 << 30) && B < 65536 && H < 65536, "sana_la_rope_apply: size out of range");
  SANA_REQUIRE(dtype == SANA_BF16 || dtype == SANA_F32, "sana_la_rope_apply: unsupported dtype");
  SANA_REQUIRE(ldq >= H * D && ldq % 8 == 0 && ldo >= H * D && ldo % 8 == 0,
               "sana_la_rope_apply: row strides must be >= H*D and multiples of 8");
  SANA_REQUIRE(aligned16(q) && aligned16(cos_table) && aligned16(sin_table) && aligned16(state) && aligned16(out),
               "sana_la_rope_apply: pointers must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define LR_APPLY(DD) lr_apply<DD>(q, ldq, cos_table, sin_table, state, out, ldo, B, N, H, eps, dtype, st)
  LR_DISPATCH(D, LR_APPLY)
#undef LR_APPLY
  return fail(SANA_ERR_INVALID, "sana_la_rope_apply: head dimension %lld", (long long)D);
}
