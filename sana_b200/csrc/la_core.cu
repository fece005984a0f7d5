// ReLU linear attention core: per-head 33x32 state reduction and apply+normalise.
//
// bf16 kernels keep one head per warp and feed warp-level bf16 tensor-core products
// (exact bf16 x bf16 products, fp32 accumulation) straight from global loads: the token /
// channel indices of the MMA fragments are permuted so that each lane's fragment registers
// are contiguous channels of a token row, so no shared-memory transpose is needed and the
// kernels are plain streaming reads at HBM speed.  fp32 kernels are FFMA (parity path).
#include <mutex>

#include "common.cuh"
#include "fp4_quant.cuh"
#include "la_plan.cuh"

namespace sana {

constexpr int HD = 32;          // head dimension (upstream linear_head_dim)
constexpr int SROWS = HD + 1;    // 32 value rows + ones row
constexpr int SSIZE = SROWS * HD;  // 1056 floats per head

constexpr int LA_WARPS = 8;  // heads per CTA

// ------------------------------------------------------------------------------------------
// state, bf16.  grid (ceil(H/8), chunks, B) - head group fastest, so that CTAs running at the
// same time read whole token rows between them; warp w -> head hg*8+w, tokens [c*Lc, min(N,(c+1)*Lc)).
// Lane (g = lane>>2, t = lane&3) loads 8 bytes = channels 4g..4g+3 of tokens n+2t, n+2t+1,
// n+2t+8, n+2t+9 for both k and v.  MMA roles: A = v^T (rows = value channel), B = relu(k).
//   A rows of M-tile mt: logical row r (<8) -> channel 4r+2mt, row r+8 -> channel 4r+2mt+1
//   B cols of N-tile nt: logical col c -> channel 4c+nt
// The ones row is a third M-tile whose A fragment is the constant "row 0 = 1".
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(LA_WARPS * 32)
la_state_bf16_kernel(const __nv_bfloat16* __restrict__ kp, const __nv_bfloat16* __restrict__ vp, int64_t ld,
                     float* __restrict__ partial, int N, int H, int Lc, int nchunks) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int h = blockIdx.x * LA_WARPS + warp;
  if (h >= H) return;
  const int b = blockIdx.z, chunk = blockIdx.y;
  const int n_begin = chunk * Lc;
  const int n_end = min(N, n_begin + Lc);

  float acc[3][4][4];
#pragma unroll
  for (int m = 0; m < 3; ++m)
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[m][n][e] = 0.f;

  const uint32_t ones = (g == 0) ? 0x3F803F80u : 0u;  // bf16 (1, 1) in logical row 0
  const int64_t col = (int64_t)h * HD + 4 * g;
  const __nv_bfloat16* kbase = kp + (int64_t)b * N * ld + col;
  const __nv_bfloat16* vbase = vp + (int64_t)b * N * ld + col;

  constexpr int U = 3;  // 16-token steps in flight per iteration
  for (int n0 = n_begin; n0 < n_end; n0 += 16 * U) {
    uint2 kr[U][4], vr[U][4];
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int tok = n0 + 16 * u + 2 * t + (i & 1) + 8 * (i >> 1);
        if (tok < n_end) {
          kr[u][i] = ldg_nc_u2(kbase + (int64_t)tok * ld);
          vr[u][i] = ldg_nc_u2(vbase + (int64_t)tok * ld);
        } else {
          kr[u][i] = make_uint2(0u, 0u);
          vr[u][i] = make_uint2(0u, 0u);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      uint32_t bfr[4][2];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        kr[u][i].x = relu_bf16x2(kr[u][i].x);
        kr[u][i].y = relu_bf16x2(kr[u][i].y);
      }
      // b0 pairs tokens (2t, 2t+1), b1 pairs tokens (2t+8, 2t+9)
      bfr[0][0] = __byte_perm(kr[u][0].x, kr[u][1].x, 0x5410);
      bfr[1][0] = __byte_perm(kr[u][0].x, kr[u][1].x, 0x7632);
      bfr[2][0] = __byte_perm(kr[u][0].y, kr[u][1].y, 0x5410);
      bfr[3][0] = __byte_perm(kr[u][0].y, kr[u][1].y, 0x7632);
      bfr[0][1] = __byte_perm(kr[u][2].x, kr[u][3].x, 0x5410);
      bfr[1][1] = __byte_perm(kr[u][2].x, kr[u][3].x, 0x7632);
      bfr[2][1] = __byte_perm(kr[u][2].y, kr[u][3].y, 0x5410);
      bfr[3][1] = __byte_perm(kr[u][2].y, kr[u][3].y, 0x7632);
      uint32_t afr[2][4];
      afr[0][0] = __byte_perm(vr[u][0].x, vr[u][1].x, 0x5410);
      afr[0][1] = __byte_perm(vr[u][0].x, vr[u][1].x, 0x7632);
      afr[0][2] = __byte_perm(vr[u][2].x, vr[u][3].x, 0x5410);
      afr[0][3] = __byte_perm(vr[u][2].x, vr[u][3].x, 0x7632);
      afr[1][0] = __byte_perm(vr[u][0].y, vr[u][1].y, 0x5410);
      afr[1][1] = __byte_perm(vr[u][0].y, vr[u][1].y, 0x7632);
      afr[1][2] = __byte_perm(vr[u][2].y, vr[u][3].y, 0x5410);
      afr[1][3] = __byte_perm(vr[u][2].y, vr[u][3].y, 0x7632);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        mma_bf16_16816(acc[0][nt], afr[0][0], afr[0][1], afr[0][2], afr[0][3], bfr[nt][0], bfr[nt][1]);
        mma_bf16_16816(acc[1][nt], afr[1][0], afr[1][1], afr[1][2], afr[1][3], bfr[nt][0], bfr[nt][1]);
        mma_bf16_16816(acc[2][nt], ones, 0u, ones, 0u, bfr[nt][0], bfr[nt][1]);
      }
    }
  }

  float* out = partial + (((int64_t)b * nchunks + chunk) * H + h) * SSIZE;
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const int i0 = 4 * g + 2 * mt;
      const int j0 = 8 * t + nt, j1 = 8 * t + 4 + nt;
      out[i0 * HD + j0] = acc[mt][nt][0];
      out[i0 * HD + j1] = acc[mt][nt][1];
      out[(i0 + 1) * HD + j0] = acc[mt][nt][2];
      out[(i0 + 1) * HD + j1] = acc[mt][nt][3];
    }
  if (g == 0) {
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      out[HD * HD + 8 * t + nt] = acc[2][nt][0];
      out[HD * HD + 8 * t + 4 + nt] = acc[2][nt][1];
    }
  }
}

// state, fp32 (FFMA).  grid (chunks, H, B), 256 threads: thread (ib = tid>>5, j = tid&31)
// owns state rows ib, ib+8, ib+16, ib+24 (and warp 0 the ones row) of column j.
__global__ void __launch_bounds__(256)
la_state_f32_kernel(const float* __restrict__ kp, const float* __restrict__ vp, int64_t ld,
                    float* __restrict__ partial, int N, int H, int Lc, int nchunks) {
  constexpr int TN = 64;
  __shared__ float ks[TN][HD];
  __shared__ float vs[TN][HD + 1];
  const int tid = threadIdx.x, j = tid & 31, ib = tid >> 5;
  const int chunk = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int n_begin = chunk * Lc, n_end = min(N, n_begin + Lc);
  const float* kbase = kp + (int64_t)b * N * ld + (int64_t)h * HD;
  const float* vbase = vp + (int64_t)b * N * ld + (int64_t)h * HD;
  float acc[5] = {0.f, 0.f, 0.f, 0.f, 0.f};
  for (int n0 = n_begin; n0 < n_end; n0 += TN) {
    __syncthreads();
    for (int e = tid; e < TN * HD; e += 256) {
      const int r = e >> 5, c = e & 31, tok = n0 + r;
      float kv = 0.f, vv = 0.f;
      if (tok < n_end) {
        kv = fmaxf(kbase[(int64_t)tok * ld + c], 0.f);
        vv = vbase[(int64_t)tok * ld + c];
      }
      ks[r][c] = kv;
      vs[r][c] = vv;
    }
    __syncthreads();
    const int lim = min(TN, n_end - n0);
    for (int r = 0; r < lim; ++r) {
      const float kv = ks[r][j];
      acc[0] = fmaf(vs[r][ib], kv, acc[0]);
      acc[1] = fmaf(vs[r][ib + 8], kv, acc[1]);
      acc[2] = fmaf(vs[r][ib + 16], kv, acc[2]);
      acc[3] = fmaf(vs[r][ib + 24], kv, acc[3]);
      acc[4] += kv;
    }
  }
  float* out = partial + (((int64_t)b * nchunks + chunk) * H + h) * SSIZE;
#pragma unroll
  for (int r = 0; r < 4; ++r) out[(ib + 8 * r) * HD + j] = acc[r];
  if (ib == 0) out[HD * HD + j] = acc[4];
}

// Adds the per-chunk partial states in chunk order (fixed order => bit-reproducible).
__global__ void la_state_reduce_kernel(const float* __restrict__ partial, float* __restrict__ state, int nchunks,
                                       int64_t per_batch /* H*SSIZE */, int64_t total /* B*H*SSIZE */) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int64_t b = idx / per_batch, r = idx - b * per_batch;
  const float* p = partial + b * nchunks * per_batch + r;
  float s = 0.f;
  for (int c = 0; c < nchunks; ++c) s += p[(int64_t)c * per_batch];
  state[idx] = s;
}

// ------------------------------------------------------------------------------------------
// apply, bf16.  grid (ceil(H/8), chunks, B); warp -> one head, 16 tokens per step.
// A = relu(q) rows (tokens), B = state^T split into bf16 hi + lo parts (two MMAs, ~2^-17
// relative error), denominator in plain fp32.  Lane (g, t) loads the 16 contiguous bytes
// q[token g (and g+8)][8t .. 8t+7]; logical K index kk of K-step s maps to channel
// 8*((kk&7)>>1) + 4s + 2*(kk>>3) + (kk&1); logical output column c of N-tile nt maps to
// value channel 8*(c>>1) + 2nt + (c&1), so each lane ends with 8 contiguous outputs of a
// row (one 16-byte store).
// ------------------------------------------------------------------------------------------
// With FP4 the kernel also - or only, when op is null - writes the NVFP4 image of its output (the input of the
// attention's output projection): a head's 32 channels of a token sit in four neighbouring lanes, eight each, so a
// 16-channel block is a lane pair; the largest magnitude produced is accumulated into sink.amax_out.
template <bool FP4>
__global__ void __launch_bounds__(LA_WARPS * 32)
la_apply_bf16_kernel(const __nv_bfloat16* __restrict__ qp, int64_t ldq, const float* __restrict__ state,
                     __nv_bfloat16* __restrict__ op, int64_t ldo, int N, int H, int Lc, float eps, const Fp4Sink sink) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int h = blockIdx.x * LA_WARPS + warp;
  if (h >= H) return;
  const int b = blockIdx.z;
  const int n_begin = blockIdx.y * Lc, n_end = min(N, n_begin + Lc);
  const float* S = state + ((int64_t)b * H + h) * SSIZE;

  uint32_t bhi[4][2][2], blo[4][2][2];
#pragma unroll
  for (int nt = 0; nt < 4; ++nt) {
    const int i = 8 * (g >> 1) + 2 * nt + (g & 1);
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      const float4 sv = *reinterpret_cast<const float4*>(S + i * HD + 8 * t + 4 * s);
      const uint32_t h0 = pack_bf16(sv.x, sv.y), h1 = pack_bf16(sv.z, sv.w);
      bhi[nt][s][0] = h0;
      bhi[nt][s][1] = h1;
      blo[nt][s][0] = pack_bf16(sv.x - bf16_lo(h0), sv.y - bf16_hi(h0));
      blo[nt][s][1] = pack_bf16(sv.z - bf16_lo(h1), sv.w - bf16_hi(h1));
    }
  }
  float sd[8];
  {
    const float4 d0 = *reinterpret_cast<const float4*>(S + HD * HD + 8 * t);
    const float4 d1 = *reinterpret_cast<const float4*>(S + HD * HD + 8 * t + 4);
    sd[0] = d0.x, sd[1] = d0.y, sd[2] = d0.z, sd[3] = d0.w;
    sd[4] = d1.x, sd[5] = d1.y, sd[6] = d1.z, sd[7] = d1.w;
  }

  const int64_t col = (int64_t)h * HD + 8 * t;
  const __nv_bfloat16* qbase = qp + (int64_t)b * N * ldq + col;
  __nv_bfloat16* obase = op + (int64_t)b * N * ldo + col;
  const float ts = FP4 ? __ldg(sink.scale_in + 1) : 0.f;
  const float inv6ts = FP4 ? __frcp_rn(6.0f * ts) : 0.f;
  float amax_local = 0.f;

  constexpr int U = 4;  // 16-token steps per batch of loads
  auto load = [&](uint4 (&qr)[U][2], int n0) {
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int tok = n0 + 16 * u + g + 8 * r;
        qr[u][r] = (tok < n_end) ? ldg_nc_u4(qbase + (int64_t)tok * ldq) : make_uint4(0u, 0u, 0u, 0u);
      }
  };
  // One batch of 16 U tokens.  As soon as a step's rows have been taken out of their registers the same rows
  // of the NEXT batch are requested into them, so the loads of a whole batch stay in flight under the products
  // without a second register set.
  auto compute = [&](uint4 (&qr)[U][2], int n0) {
    const int n_next = n0 + 16 * U;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      uint32_t a[2][4];  // [row half][word]
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        a[r][0] = relu_bf16x2(qr[u][r].x);
        a[r][1] = relu_bf16x2(qr[u][r].y);
        a[r][2] = relu_bf16x2(qr[u][r].z);
        a[r][3] = relu_bf16x2(qr[u][r].w);
      }
      if (n_next < n_end) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int tok = n_next + 16 * u + g + 8 * r;
          qr[u][r] = (tok < n_end) ? ldg_nc_u4(qbase + (int64_t)tok * ldq) : make_uint4(0u, 0u, 0u, 0u);
        }
      }
      float den[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        float d = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          d = fmaf(bf16_lo(a[r][w]), sd[2 * w], d);
          d = fmaf(bf16_hi(a[r][w]), sd[2 * w + 1], d);
        }
        d += __shfl_xor_sync(0xffffffffu, d, 1);
        d += __shfl_xor_sync(0xffffffffu, d, 2);
        den[r] = d;
      }
      float c[4][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        c[nt][0] = c[nt][1] = c[nt][2] = c[nt][3] = 0.f;
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          // K-step s: a0 = row g word 2s, a1 = row g+8 word 2s, a2 = row g word 2s+1, a3 = row g+8 word 2s+1
          mma_bf16_16816(c[nt], a[0][2 * s], a[1][2 * s], a[0][2 * s + 1], a[1][2 * s + 1], blo[nt][s][0],
                         blo[nt][s][1]);
          mma_bf16_16816(c[nt], a[0][2 * s], a[1][2 * s], a[0][2 * s + 1], a[1][2 * s + 1], bhi[nt][s][0],
                         bhi[nt][s][1]);
        }
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int tok = n0 + 16 * u + g + 8 * r;
        const bool in = tok < n_end;
        const float inv = 1.0f / (den[r] + eps);
        uint4 o;
        o.x = pack_bf16(c[0][2 * r] * inv, c[0][2 * r + 1] * inv);
        o.y = pack_bf16(c[1][2 * r] * inv, c[1][2 * r + 1] * inv);
        o.z = pack_bf16(c[2][2 * r] * inv, c[2][2 * r + 1] * inv);
        o.w = pack_bf16(c[3][2 * r] * inv, c[3][2 * r + 1] * inv);
        if (in && (!FP4 || op != nullptr)) *reinterpret_cast<uint4*>(obase + (int64_t)tok * ldo) = o;
        if (FP4) {  // every lane takes part in the shuffles; rows past the end hold zeros
          float fq[8];
          fq[0] = bf16_lo(o.x), fq[1] = bf16_hi(o.x), fq[2] = bf16_lo(o.y), fq[3] = bf16_hi(o.y);
          fq[4] = bf16_lo(o.z), fq[5] = bf16_hi(o.z), fq[6] = bf16_lo(o.w), fq[7] = bf16_hi(o.w);
          if (in) {
#pragma unroll
            for (int e = 0; e < 8; ++e) amax_local = fmaxf(amax_local, fabsf(fq[e]));
          }
          uint32_t sb;
          const uint32_t codes = fp4_quant8_of16(fq, ts, inv6ts, &sb);
          const uint32_t sb2 = __shfl_down_sync(0xffffffffu, sb, 2);
          if (in) {
            const int64_t row = (int64_t)b * N + tok;
            *reinterpret_cast<uint32_t*>(sink.q + row * (int64_t)(sink.K >> 1) + (col >> 1)) = codes;
            if (t == 0)  // the head's two 16-channel blocks: scale bytes 2h and 2h + 1 of the row
              *reinterpret_cast<uint16_t*>(sink.sf + fp4_sf_offset(row, 2 * h, sink.ktiles4)) = (uint16_t)(sb | (sb2 << 8));
          }
        }
      }
    }
  };
  uint4 qa[U][2];
  load(qa, n_begin);
#pragma unroll 1
  for (int n0 = n_begin; n0 < n_end; n0 += 16 * U) compute(qa, n0);
  if (FP4 && sink.amax_out != nullptr) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax_local = fmaxf(amax_local, __shfl_xor_sync(0xffffffffu, amax_local, o));
    if (lane == 0) atomicMax(reinterpret_cast<unsigned int*>(sink.amax_out), __float_as_uint(amax_local));  // >= 0
  }
}

// apply, fp32.  grid (chunks, H, B), 128 threads; one token per thread per step.
__global__ void __launch_bounds__(128)
la_apply_f32_kernel(const float* __restrict__ qp, int64_t ldq, const float* __restrict__ state,
                    float* __restrict__ op, int64_t ldo, int N, int H, int Lc, float eps) {
  __shared__ __align__(16) float S[SSIZE];
  const int h = blockIdx.y, b = blockIdx.z;
  const float* Sg = state + ((int64_t)b * H + h) * SSIZE;
  for (int e = threadIdx.x; e < SSIZE; e += 128) S[e] = Sg[e];
  __syncthreads();
  const int n_begin = blockIdx.x * Lc, n_end = min(N, n_begin + Lc);
  for (int tok = n_begin + threadIdx.x; tok < n_end; tok += 128) {
    const float* qrow = qp + ((int64_t)b * N + tok) * ldq + (int64_t)h * HD;
    float* orow = op + ((int64_t)b * N + tok) * ldo + (int64_t)h * HD;
    float q[HD];
#pragma unroll
    for (int v4 = 0; v4 < HD / 4; ++v4) {
      const float4 x = *reinterpret_cast<const float4*>(qrow + 4 * v4);
      q[4 * v4] = fmaxf(x.x, 0.f), q[4 * v4 + 1] = fmaxf(x.y, 0.f);
      q[4 * v4 + 2] = fmaxf(x.z, 0.f), q[4 * v4 + 3] = fmaxf(x.w, 0.f);
    }
    float den = 0.f;
#pragma unroll
    for (int jj = 0; jj < HD; ++jj) den = fmaf(S[HD * HD + jj], q[jj], den);
    den += eps;
#pragma unroll 1
    for (int i4 = 0; i4 < HD / 4; ++i4) {
      float r[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float s = 0.f;
        const float* Si = S + (4 * i4 + e) * HD;
#pragma unroll
        for (int jj = 0; jj < HD; ++jj) s = fmaf(Si[jj], q[jj], s);
        r[e] = s / den;
      }
      *reinterpret_cast<float4*>(orow + 4 * i4) = make_float4(r[0], r[1], r[2], r[3]);
    }
  }
}

static void la_state_plan(int64_t B, int64_t N, int64_t H, int dtype, int* Lc, int* nchunks) {
  // The plan must not depend on dtype-specific grids so that the workspace query needs no dtype:
  // use the bf16 head grouping (the fp32 kernel simply launches more, smaller CTAs).
  (void)dtype;
  static const int64_t slots = resident_ctas(la_state_bf16_kernel, LA_WARPS * 32);
  // a chunk's partial state (33x32 fp32, written and re-read) costs as much as 66 tokens of k+v
  la_chunking(B * ceil_div(H, LA_WARPS), N, slots, 66, Lc, nchunks);
}

}  // namespace sana

using namespace sana;

extern "C" int64_t sana_la_state_workspace_bytes(int64_t B, int64_t N, int64_t H) {
  if (B <= 0 || N <= 0 || H <= 0) return 0;
  int Lc, nchunks;
  la_state_plan(B, N, H, SANA_BF16, &Lc, &nchunks);
  return B * (int64_t)nchunks * H * SSIZE * (int64_t)sizeof(float);
}

extern "C" int sana_la_state(const void* k, const void* v, int64_t ld, float* state, void* workspace,
                             int64_t workspace_bytes, int64_t B, int64_t N, int64_t H, int dtype, void* stream) {
  SANA_REQUIRE(k && v && state && workspace, "sana_la_state: null pointer");
  SANA_REQUIRE(B > 0 && N > 0 && H > 0, "sana_la_state: B, N, H must be positive");
  SANA_REQUIRE(N < (1 << 30) && B < 65536 && H < 65536 * LA_WARPS, "sana_la_state: size out of range");
  SANA_REQUIRE(ld >= H * HD && ld % 8 == 0, "sana_la_state: ld must be >= H*32 and a multiple of 8");
  SANA_REQUIRE(aligned16(k) && aligned16(v) && aligned16(state) && aligned16(workspace),
               "sana_la_state: pointers must be 16-byte aligned");
  SANA_REQUIRE(workspace_bytes >= sana_la_state_workspace_bytes(B, N, H), "sana_la_state: workspace too small");
  int Lc, nchunks;
  la_state_plan(B, N, H, dtype, &Lc, &nchunks);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* partial = static_cast<float*>(workspace);
  if (dtype == SANA_BF16) {
    dim3 grid((unsigned)ceil_div(H, LA_WARPS), nchunks, (unsigned)B);
    la_state_bf16_kernel<<<grid, LA_WARPS * 32, 0, st>>>(static_cast<const __nv_bfloat16*>(k),
                                                        static_cast<const __nv_bfloat16*>(v), ld, partial, (int)N,
                                                        (int)H, Lc, nchunks);
  } else if (dtype == SANA_F32) {
    dim3 grid(nchunks, (unsigned)H, (unsigned)B);
    la_state_f32_kernel<<<grid, 256, 0, st>>>(static_cast<const float*>(k), static_cast<const float*>(v), ld,
                                              partial, (int)N, (int)H, Lc, nchunks);
  } else {
    return fail(SANA_ERR_UNSUPPORTED, "sana_la_state: unsupported dtype %d", dtype);
  }
  SANA_LAUNCH_CHECK("la_state kernel");
  const int64_t total = B * H * SSIZE;
  la_state_reduce_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, st>>>(partial, state, nchunks, H * SSIZE, total);
  SANA_LAUNCH_CHECK("la_state_reduce kernel");
  return SANA_OK;
}

extern "C" int sana_la_apply(const void* q, int64_t ldq, const float* state, void* out, int64_t ldo, int64_t B,
                             int64_t N, int64_t H, float eps, int dtype, void* stream) {
  SANA_REQUIRE(q && state && out, "sana_la_apply: null pointer");
  SANA_REQUIRE(B > 0 && N > 0 && H > 0, "sana_la_apply: B, N, H must be positive");
  SANA_REQUIRE(N < (1 << 30) && B < 65536 && H < 65536 * LA_WARPS, "sana_la_apply: size out of range");
  SANA_REQUIRE(ldq >= H * HD && ldq % 8 == 0 && ldo >= H * HD && ldo % 8 == 0,
               "sana_la_apply: row strides must be >= H*32 and multiples of 8");
  SANA_REQUIRE(aligned16(q) && aligned16(state) && aligned16(out), "sana_la_apply: pointers must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int Lc, nchunks;
  if (dtype == SANA_BF16) {
    static const int64_t slots = resident_ctas(la_apply_bf16_kernel<false>, LA_WARPS * 32);
    // loading a head's state costs about as much as 33 tokens of q + o
    la_chunking(B * ceil_div(H, LA_WARPS), N, slots, 33, &Lc, &nchunks);
    dim3 grid((unsigned)ceil_div(H, LA_WARPS), nchunks, (unsigned)B);
    la_apply_bf16_kernel<false><<<grid, LA_WARPS * 32, 0, st>>>(static_cast<const __nv_bfloat16*>(q), ldq, state,
                                                               static_cast<__nv_bfloat16*>(out), ldo, (int)N, (int)H, Lc,
                                                               eps, Fp4Sink{});
  } else if (dtype == SANA_F32) {
    la_chunking(B * H, N, (int64_t)sm_count() * 8, 33, &Lc, &nchunks);
    dim3 grid(nchunks, (unsigned)H, (unsigned)B);
    la_apply_f32_kernel<<<grid, 128, 0, st>>>(static_cast<const float*>(q), ldq, state, static_cast<float*>(out),
                                              ldo, (int)N, (int)H, Lc, eps);
  } else {
    return fail(SANA_ERR_UNSUPPORTED, "sana_la_apply: unsupported dtype %d", dtype);
  }
  SANA_LAUNCH_CHECK("la_apply kernel");
  return SANA_OK;
}

extern "C" int sana_la_apply_fp4(const void* q, int64_t ldq, const float* state, void* out, int64_t ldo, void* fq, void* sf,
                                 const float* scale_in, float* amax_out, int64_t B, int64_t N, int64_t H, float eps,
                                 void* stream) {
  SANA_REQUIRE(q && state && fq && sf && scale_in, "sana_la_apply_fp4: null pointer");
  SANA_REQUIRE(B > 0 && N > 0 && H > 0, "sana_la_apply_fp4: B, N, H must be positive");
  SANA_REQUIRE(N < (1 << 30) && B < 65536 && H < 65536 * LA_WARPS, "sana_la_apply_fp4: size out of range");
  SANA_REQUIRE(ldq >= H * HD && ldq % 8 == 0 && (!out || (ldo >= H * HD && ldo % 8 == 0)),
               "sana_la_apply_fp4: row strides must be >= H*32 and multiples of 8");
  SANA_REQUIRE(aligned16(q) && aligned16(state) && (!out || aligned16(out)) && aligned16(fq) && aligned16(sf),
               "sana_la_apply_fp4: pointers must be 16-byte aligned");
  Fp4Sink sink;
  sink.q = static_cast<unsigned char*>(fq);
  sink.sf = static_cast<unsigned char*>(sf);
  sink.scale_in = scale_in;
  sink.amax_out = amax_out;
  sink.K = (int)(H * HD);
  sink.ktiles4 = (int)ktiles4_of(H * HD);
  int Lc, nchunks;
  static const int64_t slots = resident_ctas(la_apply_bf16_kernel<true>, LA_WARPS * 32);
  la_chunking(B * ceil_div(H, LA_WARPS), N, slots, 33, &Lc, &nchunks);
  dim3 grid((unsigned)ceil_div(H, LA_WARPS), nchunks, (unsigned)B);
  la_apply_bf16_kernel<true><<<grid, LA_WARPS * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(q), ldq, state, static_cast<__nv_bfloat16*>(out), ldo, (int)N, (int)H, Lc, eps, sink);
  SANA_LAUNCH_CHECK("la_apply (FP4) kernel");
  return SANA_OK;
}

// ------------------------------------------------------------------------------------------
// State reduction for hosts that cannot allocate device memory.
//
// sana_la_state needs a scratch buffer for its per-chunk partial states, and somebody has to
// allocate it.  Some hosts cannot: a serving process whose device memory was carved up front
// into a fixed arena owned by another runtime, a plugin sandbox that forbids allocation
// calls, or a loop that must not hit the implicit device synchronisation of
// cudaMalloc/cudaFree while other streams are busy.  For them the scratch lives in the
// library image itself: a fixed 16 MiB array in device global memory.  Every GPU that loads
// the library carries these 16 MiB from load until the process exits, used or not.
//
// In host code the array's name is only a host-side handle, not a device address, so the
// address is fetched once per device with cudaGetSymbolAddress (that device current) and that
// pointer is what the kernels receive.
// ------------------------------------------------------------------------------------------
static __device__ __align__(256) float g_la_static_scratch[SANA_LA_STATE_NOALLOC_MAX_BYTES / sizeof(float)];

namespace sana {
static std::mutex g_scratch_mutex;
static float* g_scratch_ptr[64] = {nullptr};

// First use on a device: resolve the device address of the static scratch array.
static int static_scratch(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_status(e, "cudaGetDevice");
  if (dev < 0 || dev >= 64) return fail(SANA_ERR_UNSUPPORTED, "sana_la_state_noalloc: device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_la_static_scratch);
    if (e != cudaSuccess) return cuda_status(e, "cudaGetSymbolAddress(static scratch)");
    if (p == nullptr) return fail(SANA_ERR_DRIVER, "sana_la_state_noalloc: static scratch has no device address");
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return SANA_OK;
}
}  // namespace sana

extern "C" int sana_la_state_noalloc(const void* k, const void* v, int64_t ld, float* state, int64_t B, int64_t N,
                                     int64_t H, int dtype, void* stream) {
  SANA_REQUIRE(k && v && state, "sana_la_state_noalloc: null pointer");
  SANA_REQUIRE(B > 0 && N > 0 && H > 0, "sana_la_state_noalloc: B, N, H must be positive");
  SANA_REQUIRE(N < (1 << 30) && B < 65536 && H < 65536 * LA_WARPS, "sana_la_state_noalloc: size out of range");
  SANA_REQUIRE(ld >= H * HD && ld % 8 == 0, "sana_la_state_noalloc: ld must be >= H*32 and a multiple of 8");
  SANA_REQUIRE(aligned16(k) && aligned16(v) && aligned16(state), "sana_la_state_noalloc: pointers must be 16-byte aligned");
  SANA_REQUIRE(dtype == SANA_BF16 || dtype == SANA_F32, "sana_la_state_noalloc: unsupported dtype %d", dtype);
  const int64_t need = sana_la_state_workspace_bytes(B, N, H);
  if (need > (int64_t)SANA_LA_STATE_NOALLOC_MAX_BYTES)
    return fail(SANA_ERR_INVALID,
                "sana_la_state_noalloc: this problem needs %lld bytes of scratch but the built-in scratch holds %lld; "
                "use sana_la_state with a caller-provided workspace",
                (long long)need, (long long)SANA_LA_STATE_NOALLOC_MAX_BYTES);
  float* partial = nullptr;
  int rc = static_scratch(&partial);
  if (rc) return rc;
  int Lc, nchunks;
  la_state_plan(B, N, H, dtype, &Lc, &nchunks);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // Nothing in the scratch has to start at zero: the first launch overwrites every partial
  // state (all 1056 floats of every (batch, chunk, head)) that the second launch reads.
  if (dtype == SANA_BF16) {
    dim3 grid((unsigned)ceil_div(H, LA_WARPS), nchunks, (unsigned)B);
    la_state_bf16_kernel<<<grid, LA_WARPS * 32, 0, st>>>(static_cast<const __nv_bfloat16*>(k),
                                                        static_cast<const __nv_bfloat16*>(v), ld, partial, (int)N,
                                                        (int)H, Lc, nchunks);
  } else {
    dim3 grid(nchunks, (unsigned)H, (unsigned)B);
    la_state_f32_kernel<<<grid, 256, 0, st>>>(static_cast<const float*>(k), static_cast<const float*>(v), ld,
                                              partial, (int)N, (int)H, Lc, nchunks);
  }
  SANA_LAUNCH_CHECK("la_state kernel (static scratch)");
  const int64_t total = B * H * SSIZE;
  la_state_reduce_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, st>>>(partial, state, nchunks, H * SSIZE, total);
  SANA_LAUNCH_CHECK("la_state_reduce kernel (static scratch)");
  return SANA_OK;
}

// ------------------------------------------------------------------------------------------
// Sequence-parallel state: chunk reduction fused with the all-reduce over peer memory.
//
// Every rank owns a buffer that all ranks of the node have mapped (peer / symmetric memory):
//   [0, 256)     arrival flags: word r = last step whose state rank r has published to us
//   [256, 260)   block counter of the local launch      [320, 324) soft-error word
//   [260, 264)   exit counter, [264, 268) number of the last completed step (step = 0 in the call
//                means "the next one": the kernel numbers its steps itself, so that the same launch
//                can be replayed from a CUDA graph)
//   [1024, ...)  two state slots (step parity) of `slot_elems` floats
// One launch per step: phase A sums this rank's chunk partials into its own slot; the last
// block to finish writes `step` into its flag word on every peer (remote 4-byte stores).
// Phase B waits (bounded) until all peers' flags show `step`, then adds the ranks' slots in
// rank order - the same order everywhere, so all ranks get bit-identical totals - reading
// the peers' slots with plain loads over NVLink (no multicast, no TMA).  Slot reuse is safe
// with two parities: a rank reaches step s+1 only after every peer published step s, which
// each peer does after it finished reading step s-1.
// ------------------------------------------------------------------------------------------
namespace sana {

struct SpPeers {
  unsigned char* base[SP_MAX_WORLD];
  int rank, world;
  uint32_t step;
  int64_t slot_elems;
  long long wait_limit_ns;  // how long a block waits for the peers before it gives up
};

__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float ld_relaxed_sys_f32(const float* p) {
  float v;
  asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ long long global_ns() {
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__global__ void __launch_bounds__(256)
la_state_reduce_exchange_kernel(const float* __restrict__ partial, float* __restrict__ state, int nchunks,
                                int64_t per_batch, int64_t total, const SpPeers pg) {
  __shared__ int wait_failed;
  const int64_t first = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;  // >= total for the 32-channel heads: one element per thread
  unsigned char* mine = pg.base[pg.rank];
  // the step word only changes when the last block of a launch exits, so every block of this
  // launch reads the same value
  const uint32_t step = pg.step ? pg.step : *reinterpret_cast<volatile uint32_t*>(mine + 264) + 1u;
  const int64_t slot_off = SP_HEADER_BYTES + (int64_t)(step & 1u) * pg.slot_elems * (int64_t)sizeof(float);
  float* my_slot = reinterpret_cast<float*>(mine + slot_off);
  // ---- phase A: fixed-order sum of this rank's chunk partials, published in its slot
  for (int64_t idx = first; idx < total; idx += stride) {
    const int64_t b = idx / per_batch, r = idx - b * per_batch;
    const float* p = partial + b * nchunks * per_batch + r;
    float s = 0.f;
    for (int c = 0; c < nchunks; ++c) s += p[(int64_t)c * per_batch];
    my_slot[idx] = s;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    wait_failed = 0;
    unsigned int* counter = reinterpret_cast<unsigned int*>(mine + 256);
    const unsigned int prev = atomicAdd(counter, 1u);
    if (prev == gridDim.x - 1) {  // the whole slot is written: tell every peer
      *counter = 0u;
      __threadfence_system();
      for (int r = 0; r < pg.world; ++r)
        if (r != pg.rank) st_release_sys_u32(reinterpret_cast<uint32_t*>(pg.base[r]) + pg.rank, step);
    }
    // ---- phase B: wait for every peer's slot of this step (flags arrive in our own memory)
    const long long t0 = global_ns();
    for (int r = 0; r < pg.world && !wait_failed; ++r) {
      if (r == pg.rank) continue;
      const uint32_t* flag = reinterpret_cast<const uint32_t*>(mine) + r;
      while ((int32_t)(ld_acquire_sys_u32(flag) - step) < 0) {
        if (global_ns() - t0 > pg.wait_limit_ns) {
          wait_failed = 1;
          atomicExch(reinterpret_cast<int*>(mine + 320), 1 + r);  // which peer we gave up on
          break;
        }
      }
    }
  }
  __syncthreads();
  for (int64_t idx = first; idx < total; idx += stride) {
    const float s = my_slot[idx];  // this thread's own store of phase A
    float acc = 0.f;
    if (!wait_failed) {
      // all remote loads are issued before the first addition (each takes a few microseconds over
      // NVLink; chained behind the additions they would cost that once per peer), then the ranks'
      // values are added in rank order
      float part[SP_MAX_WORLD];
#pragma unroll
      for (int r = 0; r < SP_MAX_WORLD; ++r)
        part[r] = (r < pg.world && r != pg.rank)
                      ? ld_relaxed_sys_f32(reinterpret_cast<const float*>(pg.base[r] + slot_off) + idx)
                      : 0.f;
#pragma unroll
      for (int r = 0; r < SP_MAX_WORLD; ++r)
        if (r < pg.world) acc += (r == pg.rank) ? s : part[r];
    } else {
      acc = s;  // flagged in the soft-error word; the host must not use this result
    }
    state[idx] = acc;
  }
  if (threadIdx.x == 0) {  // the last block to leave records the step as completed
    unsigned int* exits = reinterpret_cast<unsigned int*>(mine + 260);
    if (atomicAdd(exits, 1u) == gridDim.x - 1) {
      *exits = 0u;
      *reinterpret_cast<volatile uint32_t*>(mine + 264) = step;
    }
  }
}

// Launches the kernel above on `total` state elements (`per_batch` per sample) whose chunk partials lie in
// `partial`.  Every block waits inside the kernel for the peers, and the block that finishes phase A last is the
// one that tells them, so all blocks must be resident at once: the grid is capped at what the occupancy query
// says fits (registers decide: four blocks per SM) and the threads stride over the elements.
int launch_state_reduce_exchange(const float* partial, float* state, int nchunks, int64_t per_batch, int64_t total,
                                 void* const* peer_buffers, int rank, int world, uint32_t step, cudaStream_t st) {
  SpPeers pg;
  for (int r = 0; r < world; ++r) pg.base[r] = static_cast<unsigned char*>(peer_buffers[r]);
  pg.rank = rank, pg.world = world, pg.step = step;
  pg.slot_elems = total;
  pg.wait_limit_ns = exchange_wait_limit_ns();
  int64_t blocks = ceil_div(total, 256);
  static const int64_t resident = resident_ctas(la_state_reduce_exchange_kernel, 256);
  if (blocks > resident) blocks = resident;
  la_state_reduce_exchange_kernel<<<(unsigned)blocks, 256, 0, st>>>(partial, state, nchunks, per_batch, total, pg);
  SANA_LAUNCH_CHECK("la_state_reduce_exchange kernel");
  return SANA_OK;
}

}  // namespace sana

extern "C" int64_t sana_la_state_sp_buffer_bytes(int64_t B, int64_t H) {
  if (B <= 0 || H <= 0) return 0;
  return SP_HEADER_BYTES + 2 * B * H * SSIZE * (int64_t)sizeof(float);
}

extern "C" int sana_la_state_sp(const void* k, const void* v, int64_t ld, float* state, void* workspace,
                                int64_t workspace_bytes, int64_t B, int64_t N, int64_t H, int dtype,
                                void* const* peer_buffers, int rank, int world, uint32_t step, void* stream) {
  SANA_REQUIRE(k && v && state && workspace && peer_buffers, "sana_la_state_sp: null pointer");
  SANA_REQUIRE(B > 0 && N > 0 && H > 0, "sana_la_state_sp: B, N, H must be positive");
  SANA_REQUIRE(N < (1 << 30) && B < 65536 && H < 65536 * LA_WARPS, "sana_la_state_sp: size out of range");
  SANA_REQUIRE(world >= 1 && world <= SP_MAX_WORLD && rank >= 0 && rank < world, "sana_la_state_sp: bad rank / world");
  SANA_REQUIRE(ld >= H * HD && ld % 8 == 0, "sana_la_state_sp: ld must be >= H*32 and a multiple of 8");
  SANA_REQUIRE(aligned16(k) && aligned16(v) && aligned16(state) && aligned16(workspace), "sana_la_state_sp: alignment");
  SANA_REQUIRE(workspace_bytes >= sana_la_state_workspace_bytes(B, N, H), "sana_la_state_sp: workspace too small");
  SANA_REQUIRE(dtype == SANA_BF16 || dtype == SANA_F32, "sana_la_state_sp: unsupported dtype %d", dtype);
  for (int r = 0; r < world; ++r)
    SANA_REQUIRE(peer_buffers[r] && aligned16(peer_buffers[r]), "sana_la_state_sp: peer buffer %d missing or misaligned", r);
  int Lc, nchunks;
  la_state_plan(B, N, H, dtype, &Lc, &nchunks);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* partial = static_cast<float*>(workspace);
  if (dtype == SANA_BF16) {
    dim3 grid((unsigned)ceil_div(H, LA_WARPS), nchunks, (unsigned)B);
    la_state_bf16_kernel<<<grid, LA_WARPS * 32, 0, st>>>(static_cast<const __nv_bfloat16*>(k),
                                                        static_cast<const __nv_bfloat16*>(v), ld, partial, (int)N,
                                                        (int)H, Lc, nchunks);
  } else {
    dim3 grid(nchunks, (unsigned)H, (unsigned)B);
    la_state_f32_kernel<<<grid, 256, 0, st>>>(static_cast<const float*>(k), static_cast<const float*>(v), ld,
                                              partial, (int)N, (int)H, Lc, nchunks);
  }
  SANA_LAUNCH_CHECK("la_state kernel (sequence parallel)");
  return launch_state_reduce_exchange(partial, state, nchunks, H * SSIZE, B * H * SSIZE, peer_buffers, rank, world, step, st);
}
