// Softmax core of the block's cross-attention on the tcgen05 tensor cores (bf16):
//   out[b, n, h, :] = softmax_j(q[b,n,h,:] . k[b,j,h,:] / sqrt(hd) + (1 - mask[b,j]) * -10000) v[b,j,h,:]
// for at most 304 text tokens and heads of at most 128 channels.
//
// One persistent CTA per SM walks a contiguous range of (sample, head, 128-query tile) items.
//   shared memory   K and V of the current (sample, head): [2 column blocks][LP keys][128 bytes], 128-byte
//                   swizzled, fetched by bulk-tensor copies of a 4-D view (channel, head, key, sample) so that
//                   channels past the head and keys past L arrive as zeros; one Q tile; an output staging tile.
//   tensor memory   S_A (keys [0, NA)) at column 0, S_B (keys [NA, LP)) at column 160, O at column 304.
//   warps 0-3       softmax of key chunk A: lane = query row.  Row maximum of the chunk (it fixes the row's shift m
//                   and is handed to the warps of chunk B through shared memory), p = 2^(s c - m) written back
//                   over S as bf16 pairs (the second product takes its A operand from tensor memory), row sum.
//   warps 10-13     softmax of key chunk B, on the same rows (lane quadrant = warp & 3) and the other score buffer.
//   warps 4-7       epilogue: O / row sum -> bf16 -> staging tile -> bulk-tensor store (rows past N are clipped).
//   warp 8          bulk-tensor loads (Q per tile, K / V and the mask bias per (sample, head)).
//   warp 9          one thread issues every tcgen05.mma: S_A, S_B = Q K^T, then O = P_A V_A + P_B V_B.
// The two key chunks make the pipeline: P_A V_A of tile i and S_A of tile i+1 follow the probabilities of chunk
// A, P_B V_B of tile i and S_B of tile i+1 those of chunk B.  Chunk B keeps chunk A's shift unless its own maximum
// exceeds it by more than 2^8, in which case its warps wait for P_A V_A and rescale O in tensor memory (exact
// either way: softmax is invariant to the shift, and p <= 256 is harmless in bf16 and in the fp32 accumulator);
// the factor they applied goes to the epilogue with the two partial row sums.
// Measured (20 heads x 112, 300 keys, 16 384 queries per sample): 72 - 85 us per sample, box to box (the vendor's flash kernel
// through torch: 57 - 61).  History: with ONE softmax warpgroup doing chunk A and then chunk B the kernel took 84 us:
// the 33 tcgen05.mma of a tile take about 4 500 cycles (an instruction with M = 128 costs about 130 cycles
// whether N is 112 or 256) but the softmax warps about 8 000, because a tcgen05.ld / tcgen05.st blocks the
// issuing warp for 50 - 85 cycles whether or not others are in flight and one MUFU.EX2 per element is 8.4
// cycles of the warp's scheduler (2 550 per tile).  A second warp per scheduler hides the first one's blocking
// and exponentials; splitting BY CHUNK needs one exchange per tile (the shift).  Variants that were built,
// passed the tests and were slower: a single-pass softmax with the shift fixed up on the fly (110 us); two
// warps per row splitting every chunk's columns, two exchanges per chunk (112 us); a whole chunk of the row
// held in registers to read tensor memory once instead of twice, 232 registers per softmax thread through
// setmaxnreg (104 us: ten back-to-back loads cost what ten loads hidden under the exponentials of the
// previous group cost); two query tiles in flight with 128-key chunks and direct stores (108 us: with one S
// buffer per tile a tile's softmax and its own products cannot overlap); three key chunks with three softmax
// warpgroups, or with two warpgroups taking the three chunks in turn so that a chunk's scores are requested two
// chunks ahead (94 - 95 us either way: seven more instructions on the tensor core and a third round of barriers,
// first loads and exchanges per tile); chunk A's probabilities in the tensor-memory columns behind O (chunks of 192
// + 112 keys), so that the next tile's S_A can be issued before P_A V_A, with the next query tile prefetched into
// L2 (no change: per-role cycle counters show a tile period of 7 900 cycles in which the one issuing thread is
// busy 5 500 - 33 instructions at about 167 cycles each, whatever their N - and each softmax warpgroup works 4 800
// and waits 2 800 - 3 000 for its scores, i.e. for the 16 - 17 instructions between its probabilities and its
// next scores plus whatever the other chunk has queued in front of them; the tensor pipe is the shared resource
// and it is occupied by instruction count, not by arithmetic); the whole kernel on CTA pairs (cta_group::2, M = 256,
// K and V split between the two CTAs, two Q buffers: 80 - 85 us - every SM still executes all 33 instructions of
// its own tile, so nothing is saved on the tensor pipe and the two CTAs wait for each other).  The CTAs of one launch differ by up
// to 30 % in run time with the SM they sit on, 18 % of the slowest one's time being the single-buffered Q load
// and output store (without them all CTAs run within 7 %).
// Every wait is bounded; a time-out records a code in g_cax_status and all roles leave through the teardown.
#include "tc_common.cuh"

namespace sana {

__device__ int g_cax_status = 0;

constexpr int CX_LP_MAX = 304;                       // keys, padded to a multiple of 16
constexpr int CX_KV_BLK = CX_LP_MAX * 128;           // one 64-channel block of K or V (38 912 bytes)
constexpr int CX_Q_BLK = 128 * 128;                  // one 64-channel block of a Q tile
constexpr int CX_OFF_K = 0;
constexpr int CX_OFF_V = CX_OFF_K + 2 * CX_KV_BLK;
constexpr int CX_OFF_Q = CX_OFF_V + 2 * CX_KV_BLK;
constexpr int CX_OFF_O = CX_OFF_Q + 2 * CX_Q_BLK;    // staging: [warp][block][32 rows][128 bytes]
constexpr int CX_OFF_BIAS = CX_OFF_O + 2 * CX_Q_BLK;
constexpr int CX_OFF_L = CX_OFF_BIAS + CX_LP_MAX * 4;  // per row, [4][2][128] floats: sum of chunk A, sum of chunk B,
                                                        // shift fixed by chunk A, factor chunk B put on chunk A's part
constexpr int CX_OFF_CTRL = CX_OFF_L + 4 * 2 * 128 * 4;
constexpr int CX_SMEM = CX_OFF_CTRL + 128;
constexpr int CX_THREADS = 448;  // warps 0-3 softmax of chunk A, 4-7 epilogue, 8 loads, 9 MMA issue, 10-13 softmax of chunk B
constexpr uint32_t CX_COL_SB = 160, CX_COL_O = 304;
static_assert(CX_SMEM <= 232448, "shared memory budget");
static_assert(CX_KV_BLK % 1024 == 0 && CX_OFF_Q % 1024 == 0 && CX_OFF_O % 1024 == 0, "swizzled tiles need 1024-byte bases");

struct CxArgs {
  int B, N, L, heads, hd;
  int LP, NA, NB;     // padded key count and its two chunks (multiples of 16)
  int HDN;            // hd rounded up to 16: N of the second product, K extent of the first
  int nqt;            // query tiles per (sample, head)
  int total;          // items = B * heads * nqt
  float scale_log2e;  // log2(e) / sqrt(hd)
  const __nv_bfloat16* mask;  // [B, L] of 0/1 or null
};

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(tm), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* tm, uint32_t src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               ::"l"(tm), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]: the A operand (bf16 pairs, one 32-bit column per two K indices) comes from tensor memory
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float cx_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// MN-major, 128-byte-swizzled operand (V: keys are the contraction index, channels contiguous): bits 0-13 address
// >> 4, 16-29 byte offset between 64-channel blocks (>> 4), 32-45 byte offset between 8-key groups (1024 >> 4),
// 46-47 descriptor version 1, 61-63 layout 2 (SWIZZLE_128B)
__device__ __forceinline__ uint64_t cx_desc_mn(uint32_t saddr, uint32_t block_stride_bytes) {
  const uint32_t lo = ((saddr >> 4) & 0x3FFFu) | ((block_stride_bytes >> 4) << 16);
  const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
  return ((uint64_t)hi << 32) | lo;
}

// One group of 16 scores of this lane's row (columns jb .. jb + 15 of the key axis) folded into the running maximum,
// in the scaled domain t = s * c + bias[j]; columns j >= lvalid (padding) are left out.
template <bool MASK>
__device__ __forceinline__ void cx_max16(const uint32_t (&cur)[16], float (&mx)[4], int jb, int lvalid, float c, const float* bias) {
  if (jb + 16 <= lvalid) {
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      const float s = __uint_as_float(cur[e]);
      mx[e & 3] = fmaxf(mx[e & 3], MASK ? fmaf(s, c, bias[jb + e]) : s);
    }
  } else {
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      const float s = __uint_as_float(cur[e]);
      if (jb + e < lvalid) mx[e & 3] = fmaxf(mx[e & 3], MASK ? fmaf(s, c, bias[jb + e]) : s);
    }
  }
}

// Row maximum of `ncols` scores (a multiple of 16) starting at tensor-memory address `taddr`; two register sets
// in ping-pong so that the next group's load is in flight while this one is reduced, four running maxima so that
// the comparisons do not form one long dependent chain.
template <bool MASK>
__device__ __forceinline__ float cx_row_max(uint32_t taddr, int ncols, int j0, int lvalid, float c, const float* bias) {
  float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
  uint32_t r0[16], r1[16];
  tmem_ld_32x16(taddr, r0);
  const int groups = ncols >> 4;
  for (int g = 0; g < groups; g += 2) {
    tmem_ld_wait();
    if (g + 1 < groups) tmem_ld_32x16(taddr + 16u * (uint32_t)(g + 1), r1);
    cx_max16<MASK>(r0, mx, j0 + 16 * g, lvalid, c, bias);
    if (g + 1 < groups) {
      tmem_ld_wait();
      if (g + 2 < groups) tmem_ld_32x16(taddr + 16u * (uint32_t)(g + 2), r0);
      cx_max16<MASK>(r1, mx, j0 + 16 * (g + 1), lvalid, c, bias);
    }
  }
  const float m = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
  return MASK ? m : m * c;  // c > 0
}

// p = 2^(t - m) for one group of 16 scores, written over the scores as 8 columns of bf16 pairs at `pdst`; the
// two partial row sums are updated.
template <bool MASK>
__device__ __forceinline__ void cx_exp16(const uint32_t (&cur)[16], uint32_t pdst, int jb, int lvalid, float c, float nm,
                                         const float* bias, float& sum0, float& sum1) {
  float p[16];
  if (jb + 16 <= lvalid) {
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      const float s = __uint_as_float(cur[e]);
      p[e] = cx_exp2(MASK ? fmaf(s, c, bias[jb + e] + nm) : fmaf(s, c, nm));
    }
  } else {
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      const float s = __uint_as_float(cur[e]);
      const float t = MASK ? fmaf(s, c, bias[jb + e] + nm) : fmaf(s, c, nm);  // bias holds LP entries
      p[e] = (jb + e < lvalid) ? cx_exp2(t) : 0.f;
    }
  }
  uint32_t pk[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    pk[e] = pack_bf16(p[2 * e], p[2 * e + 1]);
    sum0 += p[2 * e];
    sum1 += p[2 * e + 1];
  }
  tmem_st_32x8(pdst, pk);
}

// The same walk for the exponentials.  Group g's probabilities land on columns 8g .. 8g+7 of the chunk, whose
// scores were consumed by an earlier group (or are already in registers); the group in flight lies above them.
template <bool MASK>
__device__ __forceinline__ float cx_row_exp(uint32_t taddr, int ncols, int j0, int lvalid, float c, float m, const float* bias) {
  float sum0 = 0.f, sum1 = 0.f;
  uint32_t r0[16], r1[16];
  tmem_ld_32x16(taddr, r0);
  const int groups = ncols >> 4;
  const float nm = -m;
  for (int g = 0; g < groups; g += 2) {
    tmem_ld_wait();
    if (g + 1 < groups) tmem_ld_32x16(taddr + 16u * (uint32_t)(g + 1), r1);
    cx_exp16<MASK>(r0, taddr + 8u * (uint32_t)g, j0 + 16 * g, lvalid, c, nm, bias, sum0, sum1);
    if (g + 1 < groups) {
      tmem_ld_wait();
      if (g + 2 < groups) tmem_ld_32x16(taddr + 16u * (uint32_t)(g + 2), r0);
      cx_exp16<MASK>(r1, taddr + 8u * (uint32_t)(g + 1), j0 + 16 * (g + 1), lvalid, c, nm, bias, sum0, sum1);
    }
  }
  return sum0 + sum1;
}

template <bool MASK>
__global__ void __launch_bounds__(CX_THREADS, 1)
cross_attn_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, const CxArgs a) {
  extern __shared__ __align__(1024) unsigned char smem[];
  const uint32_t sm_u = smem_u32(smem);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if ((sm_u & 1023u) != 0u) {  // uniform over the CTA: nothing has been set up yet
    if (tid == 0) atomicExch(&g_cax_status, 9);
    return;
  }
  const uint32_t K_u = sm_u + CX_OFF_K, V_u = sm_u + CX_OFF_V, Q_u = sm_u + CX_OFF_Q, O_u = sm_u + CX_OFF_O;
  float* bias = reinterpret_cast<float*>(smem + CX_OFF_BIAS);
  float* lbuf = reinterpret_cast<float*>(smem + CX_OFF_L);
  const uint32_t ctrl = sm_u + CX_OFF_CTRL;
  // barriers (8 bytes each)
  const uint32_t bar_kv_full = ctrl, bar_kv_free = ctrl + 8, bar_q_full = ctrl + 16, bar_q_free = ctrl + 24;
  const uint32_t bar_sa = ctrl + 32, bar_sb = ctrl + 40, bar_pa = ctrl + 48, bar_pb = ctrl + 56;
  const uint32_t bar_pva = ctrl + 64, bar_o_full = ctrl + 72, bar_o_free = ctrl + 80, bar_m = ctrl + 88;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + CX_OFF_CTRL + 96);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + CX_OFF_CTRL + 100);

  // contiguous range of items for this CTA
  const int64_t t_begin = (int64_t)a.total * blockIdx.x / gridDim.x, t_end = (int64_t)a.total * (blockIdx.x + 1) / gridDim.x;
  const int n_items = (int)(t_end - t_begin);
  const int nblk = (a.HDN + 63) >> 6;  // 64-channel blocks of a head
  const int ksteps = a.HDN >> 4;       // K = 16 steps of the first product

  if (tid == 0) {
    mbar_init(bar_kv_full, 1);
    mbar_init(bar_kv_free, 1);
    mbar_init(bar_q_full, 1);
    mbar_init(bar_q_free, 1);
    mbar_init(bar_sa, 1);
    mbar_init(bar_sb, 1);
    mbar_init(bar_pa, 4);
    mbar_init(bar_pb, 4);
    mbar_init(bar_pva, 1);
    mbar_init(bar_o_full, 1);
    mbar_init(bar_o_free, 4);
    mbar_init(bar_m, 4);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmQ) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmK) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmV) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmO) : "memory");
  }
  if (warp == 9) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ctrl + 96), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 4) {
    // ------------------------------------------------------------------ softmax warps of chunk A
    // Chunk A fixes the shift m of the row and hands it to the warps of chunk B through shared memory.
    const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
    const int row = warp * 32 + lane;
    const float c = a.scale_log2e;
    uint32_t ph_sa = 0, ph_kv = 0;
    int prev_bh = -1;
    bool ok = true;
    for (int it = 0; it < n_items && ok; ++it) {
      const int bh = (int)((t_begin + it) / a.nqt);
      if (MASK && bh != prev_bh) {  // the bias vector of this sample is in shared memory once K / V have been requested
        if (!mbar_wait(bar_kv_full, ph_kv, abort_flag, 11, &g_cax_status)) { ok = false; break; }
      }
      if (bh != prev_bh) ph_kv ^= 1u;
      prev_bh = bh;
      if (!mbar_wait(bar_sa, ph_sa, abort_flag, 12, &g_cax_status)) { ok = false; break; }
      ph_sa ^= 1u;
      tcgen05_fence_after();
      const float m = cx_row_max<MASK>(lane_addr, a.NA, 0, a.L, c, bias);
      lbuf[(4 + (it & 1)) * 128 + row] = m;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_m);
      const float l = cx_row_exp<MASK>(lane_addr, a.NA, 0, a.L, c, m, bias);
      lbuf[(it & 1) * 128 + row] = l;
      tmem_st_wait();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pa);
    }
  } else if (warp >= 10) {
    // ------------------------------------------------------------------ softmax warps of chunk B
    // Same rows (warp & 3 is the lane quadrant), the other score buffer: they run beside the warps of chunk A,
    // two warps per scheduler, so that one's tensor-memory accesses and exponentials hide under the other's
    // arithmetic.  Chunk B keeps chunk A's shift unless its own maximum is more than 2^8 above it.
    const int quad = warp & 3;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    const int row = quad * 32 + lane;
    const float c = a.scale_log2e;
    uint32_t ph_sb = 0, ph_kv = 0, ph_m = 0;
    int prev_bh = -1;
    bool ok = true;
    for (int it = 0; it < n_items && ok; ++it) {
      const int bh = (int)((t_begin + it) / a.nqt);
      if (MASK && bh != prev_bh) {
        if (!mbar_wait(bar_kv_full, ph_kv, abort_flag, 11, &g_cax_status)) { ok = false; break; }
      }
      if (bh != prev_bh) ph_kv ^= 1u;
      prev_bh = bh;
      if (!mbar_wait(bar_sb, ph_sb, abort_flag, 13, &g_cax_status)) { ok = false; break; }
      ph_sb ^= 1u;
      tcgen05_fence_after();
      const float mb = cx_row_max<MASK>(lane_addr + CX_COL_SB, a.NB, a.NA, a.L, c, bias);
      if (!mbar_wait(bar_m, ph_m, abort_flag, 18, &g_cax_status)) { ok = false; break; }
      ph_m ^= 1u;
      float m = lbuf[(4 + (it & 1)) * 128 + row];
      float alpha = 1.0f;
      if (__any_sync(0xffffffffu, mb > m + 8.0f)) {
        // rare: rescale what chunk A has accumulated.  P_A V_A of this tile must have finished.
        if (!mbar_wait(bar_pva, (uint32_t)(it & 1), abort_flag, 14, &g_cax_status)) { ok = false; break; }
        tcgen05_fence_after();
        const float m_new = fmaxf(m, mb);
        alpha = cx_exp2(m - m_new);
        for (int g = 0; g < (a.HDN >> 4); ++g) {
          uint32_t o[16];
          tmem_ld_32x16(lane_addr + CX_COL_O + 16u * (uint32_t)g, o);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 16; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
          tmem_st_32x16(lane_addr + CX_COL_O + 16u * (uint32_t)g, o);
        }
        m = m_new;
      }
      const float lb = cx_row_exp<MASK>(lane_addr + CX_COL_SB, a.NB, a.NA, a.L, c, m, bias);
      lbuf[(2 + (it & 1)) * 128 + row] = lb;
      lbuf[(6 + (it & 1)) * 128 + row] = alpha;
      tmem_st_wait();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pb);
    }
  } else if (warp < 8) {
    // ------------------------------------------------------------------ epilogue warps
    const int quad = warp - 4;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + CX_COL_O;
    const int row = quad * 32 + lane;
    unsigned char* stage_row = smem + CX_OFF_O + quad * (2 * 4096) + lane * 128;  // this lane's row of block 0
    const uint32_t stage_u = O_u + (uint32_t)(quad * (2 * 4096));
    const uint32_t swz = (uint32_t)(lane & 7);
    uint32_t ph_o = 0;
    bool ok = true;
    for (int it = 0; it < n_items && ok; ++it) {
      const int64_t item = t_begin + it;
      const int bh = (int)(item / a.nqt), qt = (int)(item - (int64_t)bh * a.nqt);
      const int b = bh / a.heads, h = bh - b * a.heads;
      if (!mbar_wait(bar_o_full, ph_o, abort_flag, 15, &g_cax_status)) { ok = false; break; }
      ph_o ^= 1u;
      tcgen05_fence_after();
      const float inv = 1.0f / fmaf(lbuf[(it & 1) * 128 + row], lbuf[(6 + (it & 1)) * 128 + row], lbuf[(2 + (it & 1)) * 128 + row]);
      if (lane == 0) bulk_wait_read_all();  // the previous tile's stores have read the staging rows
      __syncwarp();
      for (int g = 0; g < (a.HDN >> 4); ++g) {
        uint32_t o[16];
        tmem_ld_32x16(lane_addr + 16u * (uint32_t)g, o);
        tmem_ld_wait();
        const int blk = g >> 2, cc = g & 3;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          float v[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(o[8 * hh + e]) * inv;
          uint4* slot = reinterpret_cast<uint4*>(stage_row + blk * 4096 + ((((uint32_t)(2 * cc + hh)) ^ swz) << 4));
          *slot = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
        }
      }
      tcgen05_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bar_o_free);  // O has been read: the next tile may overwrite it
        const int r0 = qt * 128 + quad * 32;
        if (r0 < a.N) {
          for (int blk = 0; blk < nblk; ++blk) tma_store_4d(&tmO, stage_u + (uint32_t)(blk * 4096), blk * 64, h, r0, b);
          bulk_commit();
        }
      }
    }
    if (lane == 0) bulk_wait_all();
  } else if (warp == 8) {
    // ------------------------------------------------------------------ loads
    uint32_t ph_qfree = 0, ph_kvfree = 0;
    int prev_bh = -1;
    bool ok = true;
    const uint32_t half_rows = (uint32_t)(a.LP >> 1);
    for (int it = 0; it < n_items && ok; ++it) {
      const int64_t item = t_begin + it;
      const int bh = (int)(item / a.nqt), qt = (int)(item - (int64_t)bh * a.nqt);
      const int b = bh / a.heads, h = bh - b * a.heads;
      if (it > 0) {
        if (!mbar_wait(bar_q_free, ph_qfree, abort_flag, 16, &g_cax_status)) { ok = false; break; }
        ph_qfree ^= 1u;
      }
      if (lane == 0) {
        mbar_expect_tx(bar_q_full, (uint32_t)(nblk * CX_Q_BLK));
        for (int blk = 0; blk < nblk; ++blk) tma_load_4d(Q_u + (uint32_t)(blk * CX_Q_BLK), &tmQ, bar_q_full, blk * 64, h, qt * 128, b);
      }
      if (bh != prev_bh) {
        if (prev_bh >= 0) {  // every product that reads the previous K / V (and every reader of the bias) is done
          if (!mbar_wait(bar_kv_free, ph_kvfree, abort_flag, 17, &g_cax_status)) { ok = false; break; }
          ph_kvfree ^= 1u;
        }
        if (MASK) {
          const float off = -10000.0f * 1.4426950408889634f;
          for (int j = lane; j < a.LP; j += 32)
            bias[j] = j < a.L ? (1.0f - __bfloat162float(a.mask[(int64_t)b * a.L + j])) * off : 0.f;
        }
        __syncwarp();
        if (lane == 0) {
          mbar_expect_tx(bar_kv_full, (uint32_t)(2 * nblk * a.LP * 128));
          for (int blk = 0; blk < nblk; ++blk)
            for (int hf = 0; hf < 2; ++hf) {
              const uint32_t off = (uint32_t)(blk * CX_KV_BLK) + (uint32_t)hf * half_rows * 128u;
              tma_load_4d(K_u + off, &tmK, bar_kv_full, blk * 64, h, (int)(hf * half_rows), b);
              tma_load_4d(V_u + off, &tmV, bar_kv_full, blk * 64, h, (int)(hf * half_rows), b);
            }
        }
        prev_bh = bh;
      }
    }
  } else if (warp == 9 && lane == 0) {
    // ------------------------------------------------------------------ tensor-core issue (warp 9, one thread)
    // D = f32 (bit 4), A = B = bf16 (bits 7, 10), N >> 3 at 17, M = 128 (>> 4) at 24; bit 16: B is MN-major
    const uint32_t idesc_base = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 4) << 24);
    const uint32_t idesc_sa = idesc_base | ((uint32_t)(a.NA >> 3) << 17);
    const uint32_t idesc_sb = idesc_base | ((uint32_t)(a.NB >> 3) << 17);
    const uint32_t idesc_o = idesc_base | (1u << 16) | ((uint32_t)(a.HDN >> 3) << 17);
    uint32_t ph_kv = 0, ph_q = 0, ph_pa = 0, ph_pb = 0, ph_ofree = 0;
    int prev_bh = -1;
    bool ok = true;
    auto issue_s = [&](bool chunk_b) {
      const uint32_t kbase = K_u + (chunk_b ? (uint32_t)a.NA * 128u : 0u);
      const uint32_t d = tmem_base + (chunk_b ? CX_COL_SB : 0u);
      for (int ks = 0; ks < ksteps; ++ks) {
        const uint64_t adesc = make_smem_desc(Q_u + (uint32_t)((ks >> 2) * CX_Q_BLK + (ks & 3) * 32));
        const uint64_t bdesc = make_smem_desc(kbase + (uint32_t)((ks >> 2) * CX_KV_BLK + (ks & 3) * 32));
        umma_bf16(d, adesc, bdesc, chunk_b ? idesc_sb : idesc_sa, ks != 0 ? 1u : 0u);
      }
    };
    auto issue_pv = [&](bool chunk_b) {
      const int ks_n = (chunk_b ? a.NB : a.NA) >> 4;
      const uint32_t p_tmem = tmem_base + (chunk_b ? CX_COL_SB : 0u);
      const uint64_t bdesc = cx_desc_mn(V_u + (chunk_b ? (uint32_t)a.NA * 128u : 0u), (uint32_t)CX_KV_BLK);
      for (int ks = 0; ks < ks_n; ++ks)
        umma_bf16_ts(tmem_base + CX_COL_O, p_tmem + 8u * (uint32_t)ks, bdesc + (uint64_t)(128 * ks), idesc_o,
                     (chunk_b || ks != 0) ? 1u : 0u);
    };
    for (int it = 0; it < n_items && ok; ++it) {
      const int bh = (int)((t_begin + it) / a.nqt);
      if (bh != prev_bh) {  // the pipeline was drained: start it again on the new K / V
        if (!mbar_wait(bar_kv_full, ph_kv, abort_flag, 1, &g_cax_status)) { ok = false; break; }
        ph_kv ^= 1u;
        if (!mbar_wait(bar_q_full, ph_q, abort_flag, 2, &g_cax_status)) { ok = false; break; }
        ph_q ^= 1u;
        tcgen05_fence_after();
        issue_s(false);
        umma_commit(bar_sa);
        issue_s(true);
        umma_commit(bar_sb);
        umma_commit(bar_q_free);
        prev_bh = bh;
      }
      const bool next_same = it + 1 < n_items && (int)((t_begin + it + 1) / a.nqt) == bh;
      if (!mbar_wait(bar_pa, ph_pa, abort_flag, 3, &g_cax_status)) { ok = false; break; }
      ph_pa ^= 1u;
      if (it > 0) {
        if (!mbar_wait(bar_o_free, ph_ofree, abort_flag, 4, &g_cax_status)) { ok = false; break; }
        ph_ofree ^= 1u;
      }
      tcgen05_fence_after();
      issue_pv(false);
      umma_commit(bar_pva);
      if (next_same) {
        if (!mbar_wait(bar_q_full, ph_q, abort_flag, 5, &g_cax_status)) { ok = false; break; }
        ph_q ^= 1u;
        tcgen05_fence_after();
        issue_s(false);
        umma_commit(bar_sa);
      }
      if (!mbar_wait(bar_pb, ph_pb, abort_flag, 6, &g_cax_status)) { ok = false; break; }
      ph_pb ^= 1u;
      tcgen05_fence_after();
      issue_pv(true);
      umma_commit(bar_o_full);
      if (next_same) {
        issue_s(true);
        umma_commit(bar_sb);
        umma_commit(bar_q_free);
      } else {
        umma_commit(bar_kv_free);
      }
    }
  }

  // ---------------------------------------------------------------------- teardown
  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 9) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// Whether the tensor-core kernel covers this problem (bf16 only; the caller checks the dtype).
bool cross_attn_tc_supported(int64_t L, int64_t hd) {
  return hd % 8 == 0 && hd >= 16 && hd <= 128 && L >= 17 && L <= CX_LP_MAX;
}

int cross_attn_tc_launch(const void* q, int64_t ldq, const void* k, const void* v, int64_t ldkv, const void* mask,
                         void* out, int64_t ldo, int64_t B, int64_t N, int64_t L, int heads, int hd, cudaStream_t st) {
  CxArgs a;
  a.B = (int)B, a.N = (int)N, a.L = (int)L, a.heads = heads, a.hd = hd;
  a.LP = (int)ceil_div(L, 16) * 16;
  a.NA = (int)ceil_div(a.LP / 2, 16) * 16;
  a.NB = a.LP - a.NA;
  a.HDN = (int)ceil_div(hd, 16) * 16;
  a.nqt = (int)ceil_div(N, 128);
  const int64_t total = B * heads * (int64_t)a.nqt;
  if (total >= (1LL << 31)) return fail(SANA_ERR_INVALID, "sana_cross_attention: too many query tiles");
  a.total = (int)total;
  a.scale_log2e = 1.4426950408889634f / sqrtf((float)hd);
  a.mask = static_cast<const __nv_bfloat16*>(mask);
  // 4-D views (channel, head, row, sample): channels past the head and rows past N / L are out of range
  CUtensorMap tmQ, tmK, tmV, tmO;
  auto view = [&](CUtensorMap* tm, const void* base, int64_t ld, int64_t rows, uint32_t box_rows) {
    const uint64_t dims[4] = {(uint64_t)hd, (uint64_t)heads, (uint64_t)rows, (uint64_t)B};
    const uint64_t strides[3] = {(uint64_t)hd * 2, (uint64_t)ld * 2, (uint64_t)rows * ld * 2};
    const uint32_t box[4] = {64u, 1u, box_rows, 1u};
    return make_tmap_tiled(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, base, dims, strides, box, true);
  };
  int rc = view(&tmQ, q, ldq, N, 128);
  if (rc) return rc;
  rc = view(&tmK, k, ldkv, L, (uint32_t)(a.LP / 2));
  if (rc) return rc;
  rc = view(&tmV, v, ldkv, L, (uint32_t)(a.LP / 2));
  if (rc) return rc;
  rc = view(&tmO, out, ldo, N, 32);
  if (rc) return rc;
  static OncePerDevice attr_once;
  if (attr_once.first_time()) {
    cudaError_t e = cudaFuncSetAttribute(cross_attn_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, CX_SMEM);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(cross_attn_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, CX_SMEM);
    if (e != cudaSuccess) return cuda_status(e, "cudaFuncSetAttribute(cross_attn_tc)");
  }
  const int grid = (int)(total < sm_count() ? total : sm_count());
  if (mask)
    cross_attn_tc_kernel<true><<<grid, CX_THREADS, CX_SMEM, st>>>(tmQ, tmK, tmV, tmO, a);
  else
    cross_attn_tc_kernel<false><<<grid, CX_THREADS, CX_SMEM, st>>>(tmQ, tmK, tmV, tmO, a);
  SANA_LAUNCH_CHECK("cross_attn_tc kernel");
  return SANA_OK;
}

int cross_attn_tc_take_status(int* v) {
  cudaError_t e = cudaMemcpyFromSymbol(v, g_cax_status, sizeof(int));
  if (e != cudaSuccess) return cuda_status(e, "cudaMemcpyFromSymbol(g_cax_status)");
  if (*v != 0) {
    int zero = 0;
    e = cudaMemcpyToSymbol(g_cax_status, &zero, sizeof(int));
    if (e != cudaSuccess) return cuda_status(e, "cudaMemcpyToSymbol(g_cax_status)");
  }
  return SANA_OK;
}

}  // namespace sana
