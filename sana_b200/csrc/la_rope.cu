// ReLU linear attention with a rotation of the numerator's q and k (the self-attention of
// Sana-Video): per-head (D+1) x D state reduction and apply + normalise, for heads of D channels,
// D a multiple of 16 up to 128.
//
//   state[i][j] = sum_n v[n][i] * rot(relu(k[n]))[j]   (i < D),   state[D][j] = sum_n relu(k[n][j])
//   out[n][i]   = (sum_j state[i][j] * rot(relu(q[n]))[j]) / (sum_j state[D][j] * relu(q[n][j]) + eps)
//   rot(x)[2p] = x[2p] cos[n][p] - x[2p+1] sin[n][p],  rot(x)[2p+1] = x[2p] sin[n][p] + x[2p+1] cos[n][p]
//
// bf16: one CTA per (head, token chunk, sample), 3 CTAs per SM.  The raw rows of the next 64 (state) or 32
// (apply) tokens and their cos / sin rows wait in registers while the current ones are processed; a
// staging pass applies ReLU and the rotation once per element and writes the bf16 operand tiles
// in the 128-byte-swizzled layouts the 5th-generation tensor cores read; the products are
// tcgen05.mma instructions that accumulate in tensor memory.  The key sum and the normaliser stay
// in fp32 on the CUDA cores.  fp32: plain FFMA kernels (the parity path).
#include "la_plan.cuh"
#include "tc_common.cuh"

namespace sana {

constexpr int LR_THREADS = 256;
constexpr int LR_TOK = 64;   // tokens per tile of the bf16 state kernel
constexpr int LR_TOKA = 32;  // tokens per staging sub-tile of the bf16 apply kernel
constexpr int LR_TOKF = 16;  // tokens per tile, fp32 kernels

// 16 bytes global -> shared; `valid` false writes zeros and reads nothing
__device__ __forceinline__ void lr_cp_async_16(uint32_t smem_addr, const void* gptr, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr), "l"(gptr), "r"(sz) : "memory");
}
__device__ __forceinline__ void lr_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int PENDING>
__device__ __forceinline__ void lr_cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory");
}

// ReLU of 8 bf16 channels (4 rotation pairs) of one token: x[p] = the pair relu(raw[2p], raw[2p+1])
// in fp32 (the ReLU runs on the packed bf16 pair), and rot = the rotated pairs packed back to bf16.
__device__ __forceinline__ void lr_relu_rotate8(const uint4 raw, const float4 c, const float4 s, float2 (&x)[4],
                                                uint4* rot) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  const float cc[4] = {c.x, c.y, c.z, c.w}, ss[4] = {s.x, s.y, s.z, s.w};
  uint32_t o[4];
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const uint32_t r = relu_bf16x2(w[p]);
    const float x0 = bf16_lo(r), x1 = bf16_hi(r);
    x[p] = make_float2(x0, x1);
    o[p] = pack_bf16(x0 * cc[p] - x1 * ss[p], x0 * ss[p] + x1 * cc[p]);
  }
  *rot = make_uint4(o[0], o[1], o[2], o[3]);
}

// ------------------------------------------------------------------------------------------
// state, bf16, on the 5th-generation tensor cores.  grid (H, chunks, B) - heads fastest, so that
// CTAs running at the same time read whole token rows between them.  Staging: 16 lanes per token
// (lane group `grp` owns channels 8 grp .. 8 grp + 7 and keeps their key sum in registers),
// 16 tokens per pass, 4 passes per tile.  The product sum_n v[n][i] krot[n][j] of a 64-token tile
// is four tcgen05.mma instructions (M = 128 value channels of which D are used, N = D key
// channels, K = 16 tokens each) that accumulate in tensor memory over the whole chunk.  Tokens are
// the contraction index and the tiles are token-major, i.e. both operands are "MN-major": a tile is [64-channel block][token]
// [128 bytes], 128-byte swizzled (16-byte chunk index XOR token & 7), 8-token groups 1024 bytes
// apart, channel blocks 8192 bytes apart.  v goes from global memory straight into its operand
// tile with cp.async; the conversion pass writes the rotated k into the other.
// One thread issues the products; every thread waits (bounded) for the previous tile's products
// before the tiles are overwritten.  A time-out records a code in g_lr_status, and the CTA leaves
// through the common teardown, which frees its tensor memory.
// ------------------------------------------------------------------------------------------
__device__ int g_lr_status = 0;

template <int D>
struct LrTc {
  static constexpr int BLK = LR_TOK * 128;          // one 64-channel block of a tile
  static constexpr int TILE = 2 * BLK;              // 128 channels
  static constexpr int OFF_A = TILE;                // rotated k | v[2] | control
  static constexpr int OFF_CTRL = 3 * TILE;
  static constexpr int BYTES = OFF_CTRL + 64;
  static constexpr uint32_t TMEM_COLS = 128;
  // D = f32 (bit 4), A = B = bf16 (bits 7, 10), A and B MN-major (bits 15, 16), N >> 3 at 17, M >> 4 at 24
  static constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) |
                                    ((uint32_t)(D >> 3) << 17) | ((128u >> 4) << 24);
  static_assert(TILE >= 16 * D * 4, "the key-sum scratch reuses the rotated-k tile");
};

// MN-major, 128-byte-swizzled operand: bits 0-13 address >> 4, 16-29 byte offset between 64-element
// blocks along M / N (>> 4), 32-45 byte offset between 8-row groups along K (1024 >> 4), 46-47
// descriptor version 1, 61-63 layout 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t lr_desc_mn(uint32_t saddr, uint32_t block_stride_bytes) {
  const uint32_t lo = ((saddr >> 4) & 0x3FFFu) | ((block_stride_bytes >> 4) << 16);
  const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
  return ((uint64_t)hi << 32) | lo;
}

template <int D>
__global__ void __launch_bounds__(LR_THREADS, 3)
la_rope_state_tc_kernel(const __nv_bfloat16* __restrict__ kp, const __nv_bfloat16* __restrict__ vp, int ld,
                        const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                        float* __restrict__ partial, int N, int H, int Lc, int nchunks) {
  using T = LrTc<D>;
  constexpr int G = D / 8;
  extern __shared__ __align__(1024) unsigned char smem[];
  const uint32_t sm_u = smem_u32(smem);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if ((sm_u & 1023u) != 0u) {  // uniform over the CTA: nothing has been set up yet
    if (tid == 0) atomicExch(&g_lr_status, 9);
    return;
  }
  const uint32_t B_u = sm_u, A_u = sm_u + T::OFF_A, ctrl = sm_u + T::OFF_CTRL;
  const uint32_t bar_mma = ctrl;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + T::OFF_CTRL + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + T::OFF_CTRL + 12);
  const int slot = tid >> 4, grp = tid & 15;
  const int h = blockIdx.x, chunk = blockIdx.y, b = blockIdx.z;
  const int n_begin = chunk * Lc, n_end = min(N, n_begin + Lc);
  const bool loader = grp < G;
  const int64_t col = (int64_t)h * D + 8 * grp;
  const __nv_bfloat16* kbase = kp + (int64_t)b * N * (int64_t)ld + col;
  const __nv_bfloat16* vbase = vp + (int64_t)b * N * (int64_t)ld + col;

  if (tid == 0) {
    mbar_init(bar_mma, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ctrl + 8), "r"(T::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // byte offset of (token row, 16-byte channel group) inside an operand tile
  auto tile_off = [&](int row) -> uint32_t {
    return (uint32_t)((grp >> 3) * T::BLK + row * 128 + (((grp & 7) ^ (row & 7)) << 4));
  };
  // raw k rows and their cos / sin rows of the NEXT tile wait in registers; v goes straight into its tile
  uint4 kr[LR_TOK / 16];
  float4 cr[LR_TOK / 16], sr[LR_TOK / 16];
  auto fetch = [&](int n0) {
    if (n0 + LR_TOK <= n_end) {  // whole tile (uniform): no per-row tests, nothing to clear
      if (loader) {
#pragma unroll
        for (int r = 0; r < LR_TOK / 16; ++r) {
          const int tok = n0 + 16 * r + slot;  // 32 x 32 -> 64-bit products
          kr[r] = ldg_nc_u4(kbase + (int64_t)tok * ld);
          cr[r] = __ldg(reinterpret_cast<const float4*>(cos_t + (int64_t)tok * (D / 2) + 4 * grp));
          sr[r] = __ldg(reinterpret_cast<const float4*>(sin_t + (int64_t)tok * (D / 2) + 4 * grp));
        }
      }
      return;
    }
#pragma unroll
    for (int r = 0; r < LR_TOK / 16; ++r) {
      const int tok = n0 + 16 * r + slot;
      if (loader && tok < n_end) {
        kr[r] = ldg_nc_u4(kbase + (int64_t)tok * ld);
        cr[r] = __ldg(reinterpret_cast<const float4*>(cos_t + (int64_t)tok * (D / 2) + 4 * grp));
        sr[r] = __ldg(reinterpret_cast<const float4*>(sin_t + (int64_t)tok * (D / 2) + 4 * grp));
      } else {
        kr[r] = make_uint4(0u, 0u, 0u, 0u);
        cr[r] = sr[r] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
  };
  auto issue_v = [&](int n0, int buf) {
    if (loader) {
#pragma unroll
      for (int r = 0; r < LR_TOK / 16; ++r) {
        const int row = 16 * r + slot, tok = n0 + row;
        const bool ok = tok < n_end;
        lr_cp_async_16(A_u + buf * T::TILE + tile_off(row), vbase + (int64_t)(ok ? tok : n_begin) * ld, ok);
      }
    }
    lr_cp_async_commit();
  };

  float2 ksum[4];  // packed fp32 adds
#pragma unroll
  for (int e = 0; e < 4; ++e) ksum[e] = make_float2(0.f, 0.f);

  fetch(n_begin);
  issue_v(n_begin, 0);
  bool aborted = false;
  int it = 0;
  for (int n0 = n_begin; n0 < n_end; n0 += LR_TOK, ++it) {
    const int buf = it & 1;
    // the products of the previous tile have read the rotated-k tile and v[buf ^ 1]
    // (one warp polls the barrier; the others park at the CTA barrier and spend no issue slots)
    bool ok = true;
    if (it > 0 && warp == 0) ok = mbar_wait(bar_mma, (uint32_t)((it - 1) & 1), abort_flag, 1, &g_lr_status);
    if (__syncthreads_or(!ok)) {
      aborted = true;
      break;
    }
    if (loader) {
#pragma unroll
      for (int r = 0; r < LR_TOK / 16; ++r) {
        float2 x[4];
        uint4 rot;
        lr_relu_rotate8(kr[r], cr[r], sr[r], x, &rot);
#pragma unroll
        for (int e = 0; e < 4; ++e) ksum[e] = __fadd2_rn(ksum[e], x[e]);
        *reinterpret_cast<uint4*>(smem + tile_off(16 * r + slot)) = rot;
      }
    }
    if (n0 + LR_TOK < n_end) {  // the next tile: its loads fly during this tile's products and the next wait
      fetch(n0 + LR_TOK);
      issue_v(n0 + LR_TOK, buf ^ 1);
      lr_cp_async_wait<1>();
    } else {
      lr_cp_async_wait<0>();
    }
    fence_proxy_async_smem();  // this thread's stores and completed copies, before the tensor core reads them
    __syncthreads();
    if (tid == 0) {
      tcgen05_fence_after();
      const uint64_t adesc = lr_desc_mn(A_u + buf * T::TILE, T::BLK), bdesc = lr_desc_mn(B_u, T::BLK);
#pragma unroll
      for (int k = 0; k < LR_TOK / 16; ++k)  // 16 tokens = two 8-token groups = 2048 bytes (address field is >> 4)
        umma_bf16(tmem_base, adesc + (uint64_t)(128 * k), bdesc + (uint64_t)(128 * k), T::IDESC, (it | k) != 0 ? 1u : 0u);
      umma_commit(bar_mma);
    }
  }
  lr_cp_async_wait<0>();  // nothing of this thread is still in flight, whichever way the loop ended
  if (!aborted) {
    bool ok = true;
    if (warp == 0) ok = mbar_wait(bar_mma, (uint32_t)((it - 1) & 1), abort_flag, 2, &g_lr_status);
    if (__syncthreads_or(!ok)) aborted = true;
  }
  tcgen05_fence_after();

  float* out = partial + (((int64_t)b * nchunks + chunk) * H + h) * (int64_t)((D + 1) * D);
  if (!aborted) {
    // warp w reads TMEM lanes 32 (w & 3) .. + 31 (hardware rule) = value channels, and every second
    // 16-column step = key channels
    const int quad = warp & 3, i = quad * 32 + lane;
    for (int c = warp >> 2; c < D / 16; c += 2) {
      uint32_t r[16];
      tmem_ld_32x16(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(c * 16), r);
      tmem_ld_wait();
      if (i < D) {
        float4* dst = reinterpret_cast<float4*>(out + i * D + c * 16);
#pragma unroll
        for (int e = 0; e < 4; ++e)
          dst[e] = make_float4(__uint_as_float(r[4 * e]), __uint_as_float(r[4 * e + 1]), __uint_as_float(r[4 * e + 2]),
                               __uint_as_float(r[4 * e + 3]));
      }
    }
    // key sum: the 16 token slots add in a fixed order
    float* red = reinterpret_cast<float*>(smem);  // [16][D]; the rotated-k tile is no longer read
    if (loader) {
#pragma unroll
      for (int e = 0; e < 4; ++e) *reinterpret_cast<float2*>(red + slot * D + 8 * grp + 2 * e) = ksum[e];
    }
    __syncthreads();
    if (tid < D) {
      float s = 0.f;
#pragma unroll
      for (int r = 0; r < 16; ++r) s += red[r * D + tid];
      out[D * D + tid] = s;
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 0) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(T::TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------------------------------
// apply, bf16, on the 5th-generation tensor cores.  grid (H, chunks, B).  Per tile of 128 tokens:
// out[n][i] = sum_j qrot[n][j] S[i][j] is D / 16 tcgen05.mma instructions (M = 128 tokens, N = D
// value channels, K = 16 key channels each), both operands K-major (rows of 64 channels = 128
// bytes, 128-byte swizzled, 8-row groups 1024 bytes apart, 64-channel blocks one after the other).
// The state tile is converted to bf16 once per CTA; the token tile is filled 32 tokens at a time
// by the staging pass (the next 32 tokens already in registers; ReLU + rotation as in the state
// kernel, and the 16 lanes of a token reduce its normaliser with shuffles).  Epilogue: warp w reads TMEM lanes 32 (w & 3) .. + 31 (= tokens) and every second
// 16-column step, scales by 1 / (normaliser + eps), and writes bf16 rows (padded by 16 bytes) into
// the token tile, which the products have finished reading; global stores are then 16 bytes per
// lane, 16 lanes per token.  Waits are bounded as in the state kernel.
// ------------------------------------------------------------------------------------------
constexpr int LR_MTOK = 128;  // tokens per product tile of the apply kernel

template <int D>
struct LrTcApply {
  static constexpr int KB = (D + 63) / 64;            // 64-channel blocks along the key channels
  static constexpr int S_BLK = D * 128;               // one block of the state tile: D rows x 128 bytes
  static constexpr int S_BYTES = KB * S_BLK;
  static constexpr int Q_BLK = LR_MTOK * 128;         // one block of the token tile
  static constexpr int OROWB = 2 * D + 16;            // result rows, padded
  static constexpr int Q_BYTES = (KB * Q_BLK > LR_MTOK * OROWB ? KB * Q_BLK : LR_MTOK * OROWB + 1023) / 1024 * 1024;
  static constexpr int OFF_Q = S_BYTES;               // state | tokens | key sum | 1/normaliser | control
  static constexpr int OFF_KSUM = OFF_Q + Q_BYTES;
  static constexpr int OFF_RDEN = OFF_KSUM + D * 4;
  static constexpr int OFF_CTRL = OFF_RDEN + LR_MTOK * 4;
  static constexpr int BYTES = OFF_CTRL + 64;
  static constexpr uint32_t TMEM_COLS = 128;
  // D = f32 (bit 4), A = B = bf16 (bits 7, 10), both K-major, N >> 3 at 17, M >> 4 at 24
  static constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(D >> 3) << 17) | ((128u >> 4) << 24);
  static_assert(S_BYTES % 1024 == 0 && OFF_CTRL % 8 == 0, "swizzled tiles need 1024-byte alignment");
};

template <int D>
__global__ void __launch_bounds__(LR_THREADS, 3)
la_rope_apply_tc_kernel(const __nv_bfloat16* __restrict__ qp, int ldq, const float* __restrict__ cos_t,
                        const float* __restrict__ sin_t, const float* __restrict__ state,
                        __nv_bfloat16* __restrict__ op, int ldo, int N, int H, int Lc, float eps) {
  using T = LrTcApply<D>;
  constexpr int G = D / 8;
  constexpr int SUBS = LR_MTOK / LR_TOKA;  // staging sub-tiles per product tile
  extern __shared__ __align__(1024) unsigned char smem[];
  const uint32_t sm_u = smem_u32(smem);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if ((sm_u & 1023u) != 0u) {  // uniform over the CTA: nothing has been set up yet
    if (tid == 0) atomicExch(&g_lr_status, 9);
    return;
  }
  unsigned char* Qs = smem + T::OFF_Q;
  float* ksum_s = reinterpret_cast<float*>(smem + T::OFF_KSUM);
  float* rden_s = reinterpret_cast<float*>(smem + T::OFF_RDEN);
  const uint32_t S_u = sm_u, Q_u = sm_u + T::OFF_Q, ctrl = sm_u + T::OFF_CTRL;
  const uint32_t bar_mma = ctrl;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + T::OFF_CTRL + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + T::OFF_CTRL + 12);
  const int slot = tid >> 4, grp = tid & 15;
  const int h = blockIdx.x, chunk = blockIdx.y, b = blockIdx.z;
  const int n_begin = chunk * Lc, n_end = min(N, n_begin + Lc);
  const bool loader = grp < G;
  // With two 64-channel blocks each of the 16 lane groups has a place in the token tile (the groups past the
  // head's channels fall into the tail of the rows, which the products do not read), so the lanes without
  // channels run the same loads and stores as the others on the last group's addresses and the staging pass
  // has no branches; their terms of the normaliser are multiplied by zero.
  constexpr bool ALL_LANES = T::KB == 2;
  const int lgrp = ALL_LANES ? min(grp, G - 1) : grp;
  const int64_t col = (int64_t)h * D + 8 * lgrp;
  const __nv_bfloat16* qbase = qp + (int64_t)b * N * (int64_t)ldq + col;
  __nv_bfloat16* obase = op + (int64_t)b * N * (int64_t)ldo + col;

  if (tid == 0) {
    mbar_init(bar_mma, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ctrl + 8), "r"(T::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }

  // raw q rows and their cos / sin rows of the NEXT 32 tokens wait in registers
  constexpr int RW = LR_TOKA / 16;
  uint4 qr[RW];
  float4 cr[RW], sr[RW];
#pragma unroll
  for (int r = 0; r < RW; ++r) {  // lanes without a channel group keep zeros: they join the shuffles
    qr[r] = make_uint4(0u, 0u, 0u, 0u);
    cr[r] = sr[r] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  // row r of the 32 tokens from n0; `whole`: all of them lie inside the chunk (no per-row test, nothing to clear)
  auto fetch_row = [&](int r, int n0, bool whole) {
    const int tok = n0 + 16 * r + slot;  // 32 x 32 -> 64-bit products
    if (whole ? (loader || ALL_LANES) : (loader && tok < n_end)) {
      qr[r] = ldg_nc_u4(qbase + (int64_t)tok * ldq);
      cr[r] = __ldg(reinterpret_cast<const float4*>(cos_t + (int64_t)tok * (D / 2) + 4 * lgrp));
      sr[r] = __ldg(reinterpret_cast<const float4*>(sin_t + (int64_t)tok * (D / 2) + 4 * lgrp));
    } else if (!whole) {
      qr[r] = make_uint4(0u, 0u, 0u, 0u);
      cr[r] = sr[r] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  };
#pragma unroll
  for (int r = 0; r < RW; ++r) fetch_row(r, n_begin, false);

  // the head's state as the B operand: row i (value channel), 16-byte chunks of 8 key channels
  const float* sg = state + ((int64_t)b * H + h) * (int64_t)((D + 1) * D);
  for (int e = tid; e < D * G; e += LR_THREADS) {
    const int i = e / G, c = e % G;
    const float4 lo = __ldg(reinterpret_cast<const float4*>(sg + i * D + 8 * c));
    const float4 hi = __ldg(reinterpret_cast<const float4*>(sg + i * D + 8 * c + 4));
    const uint4 pk = make_uint4(pack_bf16(lo.x, lo.y), pack_bf16(lo.z, lo.w), pack_bf16(hi.x, hi.y), pack_bf16(hi.z, hi.w));
    *reinterpret_cast<uint4*>(smem + (c >> 3) * T::S_BLK + i * 128 + (((c & 7) ^ (i & 7)) << 4)) = pk;
  }
  if (tid < D) ksum_s[tid] = __ldg(sg + D * D + tid);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  float2 kreg[4];
#pragma unroll
  for (int e = 0; e < 4; ++e)
    kreg[e] = loader ? *reinterpret_cast<const float2*>(ksum_s + 8 * grp + 2 * e) : make_float2(0.f, 0.f);

  bool aborted = false;
  int tile = 0;
  for (int m0 = n_begin; m0 < n_end; m0 += LR_MTOK, ++tile) {
    if (tile > 0) __syncthreads();  // everybody has stored the previous tile's results out of the token tile
    // the 32 tokens waiting in registers -> rows 32 ss .. of the token tile; each row's registers are asked for
    // the same row of the next 32 tokens as soon as its values have been taken out
    auto convert = [&](int ss, bool whole) {
#pragma unroll
      for (int r = 0; r < RW; ++r) {
        const int trow = ss * LR_TOKA + 16 * r + slot;
        float2 x[4];
        uint4 rot;
        lr_relu_rotate8(qr[r], cr[r], sr[r], x, &rot);
        fetch_row(r, m0 + (ss + 1) * LR_TOKA, whole);
        float2 den2 = __fmul2_rn(x[0], kreg[0]);
#pragma unroll
        for (int e = 1; e < 4; ++e) den2 = __ffma2_rn(x[e], kreg[e], den2);
        float den = den2.x + den2.y;
        // all 32 lanes take part: the 16 lanes of a token are one half of a warp
        den += __shfl_xor_sync(0xffffffffu, den, 1);
        den += __shfl_xor_sync(0xffffffffu, den, 2);
        den += __shfl_xor_sync(0xffffffffu, den, 4);
        den += __shfl_xor_sync(0xffffffffu, den, 8);
        if (grp == 0 || ALL_LANES) rden_s[trow] = __fdividef(1.0f, den + eps);  // MUFU reciprocal, 2 ulp
        if (loader || ALL_LANES)
          *reinterpret_cast<uint4*>(Qs + (grp >> 3) * T::Q_BLK + trow * 128 + (((grp & 7) ^ (trow & 7)) << 4)) = rot;
      }
    };
    if (m0 + LR_MTOK + LR_TOKA <= n_end) {  // this tile and the sub-tile after it lie inside the chunk (uniform)
#pragma unroll
      for (int ss = 0; ss < SUBS; ++ss) convert(ss, true);
    } else {
#pragma unroll 1
      for (int ss = 0; ss < SUBS; ++ss) convert(ss, false);
    }
    fence_proxy_async_smem();  // this thread's stores, before the tensor core reads them
    __syncthreads();
    if (tid == 0) {
      tcgen05_fence_after();
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {  // 16 key channels = 32 bytes inside a 128-byte row
        const uint64_t adesc = make_smem_desc(Q_u + (ks >> 2) * T::Q_BLK + (ks & 3) * 32);
        const uint64_t bdesc = make_smem_desc(S_u + (ks >> 2) * T::S_BLK + (ks & 3) * 32);
        umma_bf16(tmem_base, adesc, bdesc, T::IDESC, ks != 0 ? 1u : 0u);
      }
      umma_commit(bar_mma);
    }
    bool ok = true;  // one warp polls; the others park at the CTA barrier
    if (warp == 0) ok = mbar_wait(bar_mma, (uint32_t)(tile & 1), abort_flag, 3, &g_lr_status);
    if (__syncthreads_or(!ok)) {
      aborted = true;
      break;
    }
    tcgen05_fence_after();
    {
      const int quad = warp & 3, trow = quad * 32 + lane;
      const float rd = rden_s[trow];
      for (int c = warp >> 2; c < D / 16; c += 2) {
        uint32_t r[16];
        tmem_ld_32x16(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(c * 16), r);
        tmem_ld_wait();
        uint32_t pk[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) pk[e] = pack_bf16(__uint_as_float(r[2 * e]) * rd, __uint_as_float(r[2 * e + 1]) * rd);
        uint4* dst = reinterpret_cast<uint4*>(Qs + trow * T::OROWB + c * 32);
        dst[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        dst[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
      }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (loader) {
#pragma unroll
      for (int r = 0; r < LR_MTOK / 16; ++r) {
        const int trow = 16 * r + slot, tok = m0 + trow;
        if (tok < n_end)
          *reinterpret_cast<uint4*>(obase + (int64_t)tok * ldo) = *reinterpret_cast<const uint4*>(Qs + trow * T::OROWB + grp * 16);
      }
    }
  }
  (void)aborted;
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 0) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(T::TMEM_COLS) : "memory");
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

// Adds the per-chunk partial states in chunk order (fixed order => bit-reproducible), on top of `prior` when
// one is given (the state carried over from earlier token chunks; it may be the output buffer itself).
__global__ void la_rope_reduce_kernel(const float* __restrict__ partial, float* state, int nchunks, int64_t per_batch,
                                      int64_t total, const float* prior) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int64_t b = idx / per_batch, r = idx - b * per_batch;
  const float* p = partial + b * nchunks * per_batch + r;
  float s = prior ? prior[idx] : 0.f;
  for (int c = 0; c < nchunks; ++c) s += p[(int64_t)c * per_batch];
  state[idx] = s;
}

__global__ void add_f32_kernel(const float* a, const float* b, float* out, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = a[i] + b[i];
}

// ---- host side -------------------------------------------------------------------------------
template <int D>
struct LrSizes {
  static constexpr size_t state_tc = LrTc<D>::BYTES;
  static constexpr size_t apply_tc = LrTcApply<D>::BYTES;
  static constexpr size_t apply_f32 = ((size_t)D * (D + 1) + D + 2 * LR_TOKF * D) * 4;
};

template <int D>
static int lr_prepare() {
  static OncePerDevice once;
  if (!once.first_time()) return SANA_OK;
  cudaError_t e = cudaFuncSetAttribute(la_rope_apply_f32_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)LrSizes<D>::apply_f32);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(la_rope_apply_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)LrSizes<D>::apply_tc);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(la_rope_state_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)LrSizes<D>::state_tc);
  return cuda_status(e, "la_rope: cudaFuncSetAttribute");
}

// Chunking of the token axis.  Does not depend on dtype, so that the workspace query needs none.
template <int D>
static void lr_state_plan(int64_t B, int64_t N, int64_t H, int* Lc, int* nchunks) {
  lr_prepare<D>();  // the occupancy query needs the shared-memory attribute
  static const int64_t per_sm = resident_ctas_tmem(la_rope_state_tc_kernel<D>, LR_THREADS, LrSizes<D>::state_tc, LrTc<D>::TMEM_COLS) / sm_count();
  // a chunk's partial state ((D+1) x D fp32, written and re-read) costs as much as ~2 D tokens of k + v
  la_chunking(B * H, N, per_sm * sm_count(), 2 * D + 128, Lc, nchunks);
}

template <int D>
static int lr_state(const void* k, const void* v, int64_t ld, const float* cos_t, const float* sin_t, float* state,
                    float* partial, int64_t B, int64_t N, int64_t H, int dtype, cudaStream_t st, const float* prior,
                    void* const* peer_buffers = nullptr, int rank = 0, int world = 1, uint32_t step = 0) {
  int rc = lr_prepare<D>();
  if (rc != SANA_OK) return rc;
  int Lc, nchunks;
  lr_state_plan<D>(B, N, H, &Lc, &nchunks);
  if (dtype == SANA_BF16) {
    dim3 grid((unsigned)H, nchunks, (unsigned)B);
    la_rope_state_tc_kernel<D><<<grid, LR_THREADS, LrSizes<D>::state_tc, st>>>(
        static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), (int)ld, cos_t, sin_t, partial,
        (int)N, (int)H, Lc, nchunks);
  } else {
    dim3 grid(nchunks, (unsigned)H, (unsigned)B);
    la_rope_state_f32_kernel<D><<<grid, LR_THREADS, 0, st>>>(static_cast<const float*>(k), static_cast<const float*>(v),
                                                           ld, cos_t, sin_t, partial, (int)N, (int)H, Lc, nchunks);
  }
  SANA_LAUNCH_CHECK("la_rope_state kernel");
  const int64_t per_batch = H * (int64_t)((D + 1) * D), total = B * per_batch;
  if (peer_buffers)  // the chunk reduction does the all-reduce over the ranks' token shares as well
    return launch_state_reduce_exchange(partial, state, nchunks, per_batch, total, peer_buffers, rank, world, step, st);
  la_rope_reduce_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, st>>>(partial, state, nchunks, per_batch, total, prior);
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
        resident_ctas_tmem(la_rope_apply_tc_kernel<D>, LR_THREADS, LrSizes<D>::apply_tc, LrTcApply<D>::TMEM_COLS) / sm_count();
    // loading the head's state costs about as much as D / 2 tokens of q + out
    la_chunking(B * H, N, per_sm * sm_count(), D / 2, &Lc, &nchunks);
    dim3 grid((unsigned)H, nchunks, (unsigned)B);
    la_rope_apply_tc_kernel<D><<<grid, LR_THREADS, LrSizes<D>::apply_tc, st>>>(
        static_cast<const __nv_bfloat16*>(q), (int)ldq, cos_t, sin_t, state, static_cast<__nv_bfloat16*>(out), (int)ldo,
        (int)N, (int)H, Lc, eps);
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

static int la_rope_state_impl(const void* k, const void* v, int64_t ld, const float* cos_table, const float* sin_table,
                              const float* prior, float* state, void* workspace, int64_t workspace_bytes, int64_t B,
                              int64_t N, int64_t H, int64_t D, int dtype, void* stream, void* const* peer_buffers = nullptr,
                              int rank = 0, int world = 1, uint32_t step = 0) {
  SANA_REQUIRE(k && v && cos_table && sin_table && state && workspace, "sana_la_rope_state: null pointer");
  SANA_REQUIRE(B > 0 && N > 0 && H > 0, "sana_la_rope_state: B, N, H must be positive");
  SANA_REQUIRE(lr_head_dim_ok(D), "sana_la_rope_state: head dimension must be a multiple of 16 in [16, 128]");
  SANA_REQUIRE(N < (1 << 30) && B < 65536 && H < 65536, "sana_la_rope_state: size out of range");
  SANA_REQUIRE(dtype == SANA_BF16 || dtype == SANA_F32, "sana_la_rope_state: unsupported dtype");
  SANA_REQUIRE(ld >= H * D && ld % 8 == 0 && ld < (1LL << 31), "sana_la_rope_state: ld must be >= H*D, a multiple of 8 and below 2^31");
  SANA_REQUIRE(aligned16(k) && aligned16(v) && aligned16(cos_table) && aligned16(sin_table) && aligned16(state) &&
                   aligned16(workspace),
               "sana_la_rope_state: pointers must be 16-byte aligned");
  SANA_REQUIRE(workspace_bytes >= lr_workspace_bytes(B, N, H, D), "sana_la_rope_state: workspace too small");
  SANA_REQUIRE(!prior || aligned16(prior), "sana_la_rope_state_add: prior must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* partial = static_cast<float*>(workspace);
#define LR_STATE(DD) lr_state<DD>(k, v, ld, cos_table, sin_table, state, partial, B, N, H, dtype, st, prior, peer_buffers, rank, world, step)
  LR_DISPATCH(D, LR_STATE)
#undef LR_STATE
  return fail(SANA_ERR_INVALID, "sana_la_rope_state: head dimension %lld", (long long)D);
}

extern "C" int sana_la_rope_state(const void* k, const void* v, int64_t ld, const float* cos_table,
                                  const float* sin_table, float* state, void* workspace, int64_t workspace_bytes,
                                  int64_t B, int64_t N, int64_t H, int64_t D, int dtype, void* stream) {
  return la_rope_state_impl(k, v, ld, cos_table, sin_table, nullptr, state, workspace, workspace_bytes, B, N, H, D, dtype, stream);
}

extern "C" int sana_la_rope_state_add(const void* k, const void* v, int64_t ld, const float* cos_table,
                                      const float* sin_table, const float* prior, float* state, void* workspace,
                                      int64_t workspace_bytes, int64_t B, int64_t N, int64_t H, int64_t D, int dtype,
                                      void* stream) {
  SANA_REQUIRE(prior, "sana_la_rope_state_add: null prior");
  return la_rope_state_impl(k, v, ld, cos_table, sin_table, prior, state, workspace, workspace_bytes, B, N, H, D, dtype, stream);
}

extern "C" int64_t sana_la_rope_state_sp_buffer_bytes(int64_t B, int64_t H, int64_t D) {
  if (B <= 0 || H <= 0 || !lr_head_dim_ok(D)) return 0;
  return SP_HEADER_BYTES + 2 * B * H * (D + 1) * D * (int64_t)sizeof(float);
}

extern "C" int sana_la_rope_state_sp(const void* k, const void* v, int64_t ld, const float* cos_table,
                                     const float* sin_table, float* state, void* workspace, int64_t workspace_bytes,
                                     int64_t B, int64_t N, int64_t H, int64_t D, int dtype, void* const* peer_buffers,
                                     int rank, int world, uint32_t step, void* stream) {
  SANA_REQUIRE(peer_buffers, "sana_la_rope_state_sp: null pointer");
  SANA_REQUIRE(world >= 1 && world <= SP_MAX_WORLD && rank >= 0 && rank < world, "sana_la_rope_state_sp: bad rank / world");
  for (int r = 0; r < world; ++r)
    SANA_REQUIRE(peer_buffers[r] && aligned16(peer_buffers[r]), "sana_la_rope_state_sp: peer buffer %d missing or misaligned", r);
  return la_rope_state_impl(k, v, ld, cos_table, sin_table, nullptr, state, workspace, workspace_bytes, B, N, H, D, dtype,
                            stream, peer_buffers, rank, world, step);
}

extern "C" int sana_add_f32(const float* a, const float* b, float* out, int64_t n, void* stream) {
  SANA_REQUIRE(a && b && out && n > 0, "sana_add_f32: bad arguments");
  add_f32_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(a, b, out, n);
  SANA_LAUNCH_CHECK("add_f32 kernel");
  return SANA_OK;
}

extern "C" int sana_la_rope_apply(const void* q, int64_t ldq, const float* cos_table, const float* sin_table,
                                  const float* state, void* out, int64_t ldo, int64_t B, int64_t N, int64_t H,
                                  int64_t D, float eps, int dtype, void* stream) {
  SANA_REQUIRE(q && cos_table && sin_table && state && out, "sana_la_rope_apply: null pointer");
  SANA_REQUIRE(B > 0 && N > 0 && H > 0, "sana_la_rope_apply: B, N, H must be positive");
  SANA_REQUIRE(lr_head_dim_ok(D), "sana_la_rope_apply: head dimension must be a multiple of 16 in [16, 128]");
  SANA_REQUIRE(N < (1 << 30) && B < 65536 && H < 65536, "sana_la_rope_apply: size out of range");
  SANA_REQUIRE(dtype == SANA_BF16 || dtype == SANA_F32, "sana_la_rope_apply: unsupported dtype");
  SANA_REQUIRE(ldq >= H * D && ldq % 8 == 0 && ldo >= H * D && ldo % 8 == 0 && ldq < (1LL << 31) && ldo < (1LL << 31),
               "sana_la_rope_apply: row strides must be >= H*D, multiples of 8 and below 2^31");
  SANA_REQUIRE(aligned16(q) && aligned16(cos_table) && aligned16(sin_table) && aligned16(state) && aligned16(out),
               "sana_la_rope_apply: pointers must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define LR_APPLY(DD) lr_apply<DD>(q, ldq, cos_table, sin_table, state, out, ldo, B, N, H, eps, dtype, st)
  LR_DISPATCH(D, LR_APPLY)
#undef LR_APPLY
  return fail(SANA_ERR_INVALID, "sana_la_rope_apply: head dimension %lld", (long long)D);
}

extern "C" int sana_la_rope_take_device_status(int* status_out) {
  if (!status_out) return fail(SANA_ERR_INVALID, "sana_la_rope_take_device_status: null pointer");
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_lr_status, sizeof(int));
  if (e != cudaSuccess) return cuda_status(e, "cudaMemcpyFromSymbol(g_lr_status)");
  if (v != 0) {
    const int zero = 0;
    e = cudaMemcpyToSymbol(g_lr_status, &zero, sizeof(int));
    if (e != cudaSuccess) return cuda_status(e, "cudaMemcpyToSymbol(g_lr_status)");
  }
  *status_out = v;
  return SANA_OK;
}
