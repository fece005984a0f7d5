// NVFP4 projection: out = epilogue(a_scale * w_scale * (Aq . SFa) @ (Wq . SFw)^T).
//
// Operands are E2M1 values packed two per byte (K-major), with one E4M3 scale per 16
// consecutive K elements and one fp32 scale per tensor.  The block scales live in global
// memory in the 512-byte tiles the tensor core consumes: tile (row block of 128, K block of
// 64) holds byte [(r % 32) * 16 + (r / 32) * 4 + kb] for row r and 16-element block kb; tiles
// are ordered K-fastest and the K-tile count is padded to a multiple of 4, so one pipeline
// stage (K = 256) needs 2 KiB contiguous scale bytes per operand.
//
// Same persistent, warp-specialised structure as the bf16 kernel (128 x 128 tiles, K = 256
// per stage): the producer adds two bulk copies for the scale tiles, the MMA lane copies
// them from shared to tensor memory (tcgen05.cp 32x128b.warpx4 replicates each 512-byte tile
// over the four lane quadrants) and issues tcgen05.mma kind::mxf4nvf4 with block-16 scales,
// K = 64 per instruction.  TMEM: two 128-column accumulators + 32 scale columns per stage.
#include <cuda_fp8.h>

#include "fp4_quant.cuh"
#include "tc_common.cuh"

namespace sana {

__device__ int g_fp4_status = 0;

constexpr int F4_BM = 128, F4_BN = 128;
constexpr int F4_BK = 256;                          // elements per stage = 128 bytes per row
constexpr int F4_A_BYTES = F4_BM * 128;             // 16 KiB
constexpr int F4_B_BYTES = F4_BN * 128;             // 16 KiB
constexpr int F4_SF_BYTES = 4 * 512;                // four 512-byte scale tiles per operand and stage
constexpr int F4_STAGE_BYTES = F4_A_BYTES + F4_B_BYTES + 2 * F4_SF_BYTES;  // 36 KiB
constexpr int F4_STAGES = 5;
constexpr int F4_CTRL_BYTES = 256;
constexpr int F4_EPI_WARPS = 8;
constexpr int F4_EPI_BYTES = F4_EPI_WARPS * EPI_BOX_BYTES;  // one 32 x 64 box per epilogue warp (tc_common.cuh)
constexpr int F4_SMEM_BYTES = F4_STAGES * F4_STAGE_BYTES + F4_EPI_BYTES + F4_CTRL_BYTES;
static_assert(16 * F4_STAGES + 40 + 8 * F4_EPI_WARPS <= F4_CTRL_BYTES, "control block too small");
constexpr int F4_THREADS = 64 + 32 * F4_EPI_WARPS;
constexpr int F4_TMEM_COLS = 512;                   // 2 x 128 accumulator + 6 x 32 scale columns = 448
constexpr int F4_SF_COL0 = 2 * F4_BN;               // first scale column
// block-scaled instruction descriptor: A = B = E2M1 (code 1 at bits 7 and 10), both K-major,
// scale type UE4M3 (bit 23 = 0), N>>3 at bit 17, M>>4 at bit 24, dense K = 64 (bit 31 = 0)
constexpr uint32_t F4_IDESC = (1u << 7) | (1u << 10) | ((uint32_t)(F4_BN >> 3) << 17) | ((uint32_t)(F4_BM >> 4) << 24);
static_assert(F4_SMEM_BYTES <= 232448, "shared memory budget");

__device__ __forceinline__ void bulk_load(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_dst),
               "l"(gsrc), "r"(bytes), "r"(bar)
               : "memory");
}

// 32 rows x 16 bytes, rows contiguous: 8-row groups 128 bytes apart, no swizzle
__device__ __forceinline__ uint64_t make_sf_desc(uint32_t saddr) {
  const uint32_t lo = (saddr >> 4) & 0x3FFFu;
  const uint32_t hi = (128u >> 4) | (1u << 14);
  return ((uint64_t)hi << 32) | lo;
}

__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

__device__ __forceinline__ void umma_nvfp4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa,
                                           uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
      : "memory");
}

struct F4Args {
  __nv_bfloat16* out;
  int64_t ldo;
  const unsigned char* sfa;   // scale tiles of A: [ceil(M/128)][ktiles4][512]
  const unsigned char* sfb;   // scale tiles of W: [ceil(N/128)][ktiles4][512]
  const float* a_scale;       // per-tensor scales (device)
  const float* w_scale;
  int M, N, K;
  int tiles_m, tiles_n;
  int ktiles4;                // K tiles of 64 per row block, padded to a multiple of 4
  EpiParams ep;
};

__global__ void __launch_bounds__(F4_THREADS, 1)
gemm_nvfp4_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const __grid_constant__ CUtensorMap tmOut, const __grid_constant__ CUtensorMap tmRes,
                     const F4Args args) {
  constexpr int STAGES = F4_STAGES;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t tiles_base = smem_u32(smem_raw);
  const uint32_t epi_base = tiles_base + STAGES * F4_STAGE_BYTES;  // staging boxes of the epilogue warps
  unsigned char* epi_gen = smem_raw + STAGES * F4_STAGE_BYTES;
  const uint32_t ctrl = epi_base + F4_EPI_BYTES;
  unsigned char* ctrl_gen = epi_gen + F4_EPI_BYTES;
  // control layout: full[STAGES] | empty[STAGES] | tfull[2] | tempty[2] | tmem ptr | abort | res[EPI_WARPS]
  const uint32_t bar_full = ctrl, bar_empty = ctrl + 8 * STAGES;
  const uint32_t bar_tfull = ctrl + 16 * STAGES, bar_tempty = bar_tfull + 16;
  const uint32_t bar_res = ctrl + 16 * STAGES + 40;
  volatile uint32_t* tmem_ptr_slot = reinterpret_cast<volatile uint32_t*>(ctrl_gen + 16 * STAGES + 32);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(ctrl_gen + 16 * STAGES + 36);

  if ((tiles_base & 1023u) != 0u) {
    if (threadIdx.x == 0) atomicExch(&g_fp4_status, 9);
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = args.tiles_m * args.tiles_n;
  const int kblocks = (args.K + F4_BK - 1) / F4_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, F4_EPI_WARPS);
    }
    for (int w = 0; w < F4_EPI_WARPS; ++w) mbar_init(bar_res + 8 * w, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmA) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmOut) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmRes) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ctrl + 16 * STAGES + 32),
                 "r"((uint32_t)F4_TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_ptr_slot;

  if (warp == 0) {
    // ------------------------------- producer -----------------------------------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int mt = tile / args.tiles_n, nt = tile % args.tiles_n;
        const unsigned char* sfa_row = args.sfa + (int64_t)mt * args.ktiles4 * 512;
        const unsigned char* sfb_row = args.sfb + (int64_t)nt * args.ktiles4 * 512;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, 1, &g_fp4_status)) { ok = false; break; }
          const uint32_t sa = tiles_base + stage * F4_STAGE_BYTES;
          const uint32_t fb = bar_full + 8 * stage;
          mbar_expect_tx(fb, F4_STAGE_BYTES);
          tma_load_2d(sa, &tmA, fb, kb * 128, mt * F4_BM);                 // byte coordinates along K
          tma_load_2d(sa + F4_A_BYTES, &tmB, fb, kb * 128, nt * F4_BN);
          bulk_load(sa + F4_A_BYTES + F4_B_BYTES, sfa_row + (int64_t)kb * F4_SF_BYTES, F4_SF_BYTES, fb);
          bulk_load(sa + F4_A_BYTES + F4_B_BYTES + F4_SF_BYTES, sfb_row + (int64_t)kb * F4_SF_BYTES, F4_SF_BYTES, fb);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ---------------------------------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      uint32_t acc_phase = 0u;
      bool ok = true;
      int it = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
        const int a = it & 1;
        if (!mbar_wait(bar_tempty + 8 * a, ((acc_phase >> a) & 1u) ^ 1u, abort_flag, 2, &g_fp4_status)) { ok = false; break; }
        acc_phase ^= 1u << a;
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(a * F4_BN);
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, 3, &g_fp4_status)) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t sa = tiles_base + stage * F4_STAGE_BYTES;
          const uint64_t adesc = make_smem_desc(sa), bdesc = make_smem_desc(sa + F4_A_BYTES);
          const uint32_t sfa_s = sa + F4_A_BYTES + F4_B_BYTES, sfb_s = sfa_s + F4_SF_BYTES;
          const uint32_t sfa_t = tmem_base + (uint32_t)(F4_SF_COL0 + stage * 32), sfb_t = sfa_t + 16;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            tmem_cp_sf(sfa_t + 4 * k, make_sf_desc(sfa_s + 512 * k));
            tmem_cp_sf(sfb_t + 4 * k, make_sf_desc(sfb_s + 512 * k));
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            // 64 elements = 32 bytes per instruction inside the 128-byte swizzle row
            umma_nvfp4(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), F4_IDESC, sfa_t + 4 * k, sfb_t + 4 * k,
                       (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(bar_empty + 8 * stage);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(bar_tfull + 8 * a);
      }
    }
  } else {
    // ------------------------------- epilogue warps -----------------------------------
    // staged epilogue (tc_common.cuh): a warp owns 32 rows x 64 columns = one box
    const int ew = warp - 2;
    const int quad = warp & 3;
    const int half = ew >> 2;
    constexpr int HALF = F4_BN / 2, NCHUNK = HALF / 16;
    static_assert(HALF == EPI_BOX_COLS, "one staging box per epilogue warp");
    const EpiParams& ep = args.ep;
    const int64_t N = args.N;
    const bool has_res = ep.residual != nullptr;
    const float alpha = __ldg(args.a_scale) * __ldg(args.w_scale);
    EpiBox eb;
    eb.box_s = epi_base + (uint32_t)(ew * EPI_BOX_BYTES);
    eb.row_g = epi_gen + ew * EPI_BOX_BYTES + lane * 128;
    eb.res_bar = bar_res + 8 * ew;
    eb.res_phase = 0u;
    eb.swz = (uint32_t)(lane & 7);
    uint32_t full_phase = 0u;
    bool ok = true;
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
      const int a = it & 1;
      const int m_box = (tile / args.tiles_n) * F4_BM + quad * 32;
      const int64_t nbase = (int64_t)(tile % args.tiles_n) * F4_BN + half * HALF;
      const int64_t m = (int64_t)m_box + lane;
      const bool row_ok = m < args.M;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(a * F4_BN + half * HALF);
      const EpiRow row = epi_row_setup(ep, m, row_ok, nbase, N);
      const bool box_rows_in = m_box < args.M;
      const bool use_res = has_res && box_rows_in;
      epi_box_begin<1>(eb, row, use_res, lane, m_box, &tmRes);
      EpiStep st[2];
      epi_fetch(row, st[0], 0);  // operands that do not depend on the accumulator: requested before the wait
      if (!mbar_wait(bar_tfull + 8 * a, (full_phase >> a) & 1u, abort_flag, 4, &g_fp4_status)) { ok = false; break; }
      full_phase ^= 1u << a;
      tcgen05_fence_after();
      if (!epi_box_drain<NCHUNK, true>(eb, row, ep, taddr, st, use_res, box_rows_in, lane, m_box, &tmOut, alpha,
                                       abort_flag, &g_fp4_status)) {
        ok = false;
        break;
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + 8 * a);
    }
    if (lane == 0) bulk_wait_all();  // the boxes stay valid until the last stores have drained
  }

  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)F4_TMEM_COLS)
                 : "memory");
  }
}


// ---- CTA-pair variant -----------------------------------------------------------------------------
// Two CTAs of a cluster share one 256 x 256 output tile (tcgen05 cta_group::2): each CTA loads its own
// 128 rows of A with their scale tiles, HALF of the W tile (128 rows) and the scale tiles of the whole W
// tile; the pair's leader copies the scales into tensor memory and issues the block-scaled MMAs with
// M = 256.  A block-scaled MMA of K = 64 takes the tensor core about as long for a 128 x 128 tile as for
// a 256 x 256 one (measured: 262 / 290 / 305 cycles per instruction on 128 x 128, 256 x 128, 256 x 256),
// so only the largest tile uses it fully.  Tensor memory then holds ONE 256-column accumulator (two would
// leave no room for the scale columns).  To keep its epilogue off the critical path the epilogue warps
// first copy the whole accumulator into registers (eight back-to-back tcgen05.ld per warp, a few hundred
// cycles), hand the buffer back to the MMA issuer, and do the arithmetic and the stores from registers
// under the next tile's MMAs; they get the registers for that from the load / MMA warps (setmaxnreg).
// All four operand streams are bulk-tensor copies (the scale buffers as [tiles, 128] words, so that
// tiles past the end arrive as zeros), counted on the leader's barrier.  Roles of warpgroup 0: warp 0 loads,
// warp 1 issues the MMAs, warp 2 issues the scale copies (a third of the tensor pipe's time when they sat in
// the MMA thread's instruction stream), warp 3 idle.  Output tiles are walked in groups of eight tile rows.
constexpr int P4_BM = 128, P4_BN = 256;
constexpr int P4_A_BYTES = P4_BM * 128;             // 16 KiB
constexpr int P4_B_BYTES = (P4_BN / 2) * 128;       // 16 KiB: this CTA's half of the W tile
constexpr int P4_SFA_BYTES = 4 * 512;               // scale tiles of this CTA's A rows, K = 256
constexpr int P4_SFB_BYTES = 2 * 4 * 512;           // scale tiles of all 256 W rows
constexpr int P4_STAGE_BYTES = P4_A_BYTES + P4_B_BYTES + P4_SFA_BYTES + P4_SFB_BYTES;  // 38 KiB
constexpr int P4_STAGES = 4;
constexpr int P4_EPI_WARPS = 8;
constexpr int P4_NBOX = (P4_BN / 2) / EPI_BOX_COLS;  // staging boxes per epilogue warp
constexpr int P4_EPI_BYTES = P4_EPI_WARPS * P4_NBOX * EPI_BOX_BYTES;
constexpr int P4_CTRL_BYTES = 256;
constexpr int P4_SMEM_BYTES = P4_STAGES * P4_STAGE_BYTES + P4_EPI_BYTES + P4_CTRL_BYTES;
constexpr int P4_THREADS = 128 + 32 * P4_EPI_WARPS;  // warpgroup 0: loads, MMA, two idle warps; then the epilogue warps
constexpr int P4_SF_COL0 = P4_BN;                   // scale columns follow the accumulator
constexpr int P4_SF_COLS = 16 + 32;                 // per stage: A 4 x 4, W 4 x 8
constexpr uint32_t P4_IDESC = (1u << 7) | (1u << 10) | ((uint32_t)(P4_BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
static_assert(P4_SMEM_BYTES <= 232448, "shared memory budget");
static_assert(P4_STAGE_BYTES % 1024 == 0, "stage bases must stay 1024-byte aligned");
static_assert(P4_SF_COL0 + P4_STAGES * P4_SF_COLS <= 512, "tensor memory budget");
static_assert(16 * P4_STAGES + 40 + 8 * P4_EPI_WARPS + 8 * P4_STAGES <= P4_CTRL_BYTES, "control block too small");

__device__ __forceinline__ void tmem_cp_sf_pair(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// arrive (once, on this CTA's barrier) when every tcgen05 operation this thread has issued so far is complete
__device__ __forceinline__ void tc_commit_pair_local(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void umma_nvfp4_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa,
                                                uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
      : "memory");
}

struct P4Args {
  __nv_bfloat16* out;
  int64_t ldo;
  const float* a_scale;
  const float* w_scale;
  int M, N, K;
  int tiles_m, tiles_n;  // 256 x 256 pair tiles
  int ktiles4;
  EpiParams ep;
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P4_THREADS, 1)
gemm_nvfp4_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                       const __grid_constant__ CUtensorMap tmSFA, const __grid_constant__ CUtensorMap tmSFB,
                       const __grid_constant__ CUtensorMap tmOut, const __grid_constant__ CUtensorMap tmRes,
                       const P4Args args) {
  constexpr int STAGES = P4_STAGES;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t tiles_base = smem_u32(smem_raw);
  const uint32_t epi_base = tiles_base + STAGES * P4_STAGE_BYTES;
  unsigned char* epi_gen = smem_raw + STAGES * P4_STAGE_BYTES;
  const uint32_t ctrl = epi_base + P4_EPI_BYTES;
  unsigned char* ctrl_gen = epi_gen + P4_EPI_BYTES;
  // control layout: full[STAGES] | empty[STAGES] | tfull | (pad) | tempty | (pad) | tmem ptr | abort | res[EPI_WARPS] | sf[STAGES]
  const uint32_t bar_full = ctrl, bar_empty = ctrl + 8 * STAGES;
  const uint32_t bar_tfull = ctrl + 16 * STAGES, bar_tempty = bar_tfull + 16;
  const uint32_t bar_res = ctrl + 16 * STAGES + 40;
  const uint32_t bar_sf = bar_res + 8 * P4_EPI_WARPS;  // leader only: the scale copies of a stage have landed in tensor memory
  volatile uint32_t* tmem_ptr_slot = reinterpret_cast<volatile uint32_t*>(ctrl_gen + 16 * STAGES + 32);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(ctrl_gen + 16 * STAGES + 36);

  if ((tiles_base & 1023u) != 0u) {  // cluster-uniform: the dynamic window starts at the same offset in every CTA
    if (threadIdx.x == 0) atomicExch(&g_fp4_status, 9);
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  const int num_tiles = args.tiles_m * args.tiles_n;
  const int kblocks = (args.K + F4_BK - 1) / F4_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
      mbar_init(bar_sf + 8 * s, 1);
    }
    mbar_init(bar_tfull, 1);
    mbar_init(bar_tempty, 2 * P4_EPI_WARPS);
    for (int w = 0; w < P4_EPI_WARPS; ++w) mbar_init(bar_res + 8 * w, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmA) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmSFA) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmSFB) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmOut) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmRes) : "memory");
  }
  if (warp == 1) {  // the same warp of both CTAs allocates collectively
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ctrl + 16 * STAGES + 32), "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything signals them
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_ptr_slot;
  // 384 threads start with 168 registers each; the epilogue warps, which hold a 128-column slice of the
  // accumulator, take over what warpgroup 0 (loads, MMA issue, two idle warps) gives up
  if (warp < 4) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
  if (warp == 0) {
    // ------------------------------- loads (both CTAs) ----------------------------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      const uint32_t full0 = map_to_cta(bar_full, 0);  // the leader's full barriers, cluster address
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        int mt, nt;
        pair_tile_coords(tile, args.tiles_m, args.tiles_n, mt, nt);
        const int m0 = mt * 256 + (int)rank * P4_BM;          // this CTA's A rows
        const int n0 = nt * P4_BN + (int)rank * (P4_BN / 2);  // this CTA's half of the W rows
        const int sfa_row = (2 * mt + (int)rank) * args.ktiles4;  // scale tiles: row blocks of 128, K-fastest
        const int sfb_row = (2 * nt) * args.ktiles4;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, 1, &g_fp4_status)) { ok = false; break; }
          const uint32_t sa = tiles_base + stage * P4_STAGE_BYTES;
          if (leader) mbar_expect_tx(bar_full + 8 * stage, 2 * P4_STAGE_BYTES);
          const uint32_t fb = full0 + 8 * stage;
          tma_load_2d_pair(sa, &tmA, fb, kb * 128, m0);  // byte coordinates along K
          tma_load_2d_pair(sa + P4_A_BYTES, &tmB, fb, kb * 128, n0);
          tma_load_2d_pair(sa + P4_A_BYTES + P4_B_BYTES, &tmSFA, fb, 0, sfa_row + 4 * kb);
          tma_load_2d_pair(sa + P4_A_BYTES + P4_B_BYTES + P4_SFA_BYTES, &tmSFB, fb, 0, sfb_row + 4 * kb);
          tma_load_2d_pair(sa + P4_A_BYTES + P4_B_BYTES + P4_SFA_BYTES + 4 * 512, &tmSFB, fb, 0, sfb_row + args.ktiles4 + 4 * kb);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (leader CTA only) -----------------------
    if (leader && lane == 0) {
      uint32_t stage = 0, phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        if (!mbar_wait(bar_tempty, acc_phase ^ 1u, abort_flag, 2, &g_fp4_status)) { ok = false; break; }
        acc_phase ^= 1u;
        tcgen05_fence_after();
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, 3, &g_fp4_status)) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t sa = tiles_base + stage * P4_STAGE_BYTES;
          const uint64_t adesc = make_smem_desc(sa), bdesc = make_smem_desc(sa + P4_A_BYTES);
          const uint32_t sfa_t = tmem_base + (uint32_t)(P4_SF_COL0 + stage * P4_SF_COLS), sfb_t = sfa_t + 16;
          // the stage's scales are copied into tensor memory by warp 2, off this thread's instruction stream
          if (!mbar_wait(bar_sf + 8 * stage, phase, abort_flag, 6, &g_fp4_status)) { ok = false; break; }
          tcgen05_fence_after();
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_nvfp4_pair(tmem_base, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), P4_IDESC, sfa_t + 4 * k,
                            sfb_t + 8 * k, (kb | k) != 0 ? 1u : 0u);
          umma_commit_pair(bar_empty + 8 * stage);  // frees this stage in both CTAs
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit_pair(bar_tfull);  // accumulator complete, both CTAs
      }
    }
  } else if (warp == 2) {
    // ------------------------------- scale copies (leader CTA only) ----------------------
    // Twelve tcgen05.cp per stage move the stage's scale tiles from shared into tensor memory (each CTA's own
    // tiles into its own tensor memory).  Issued by the MMA thread they sit between its MMAs in program order;
    // from a thread of their own they run ahead, under the MMAs of the stage before.
    if (leader && lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, 7, &g_fp4_status)) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t sa = tiles_base + stage * P4_STAGE_BYTES;
          const uint32_t sfa_s = sa + P4_A_BYTES + P4_B_BYTES, sfb_s = sfa_s + P4_SFA_BYTES;
          const uint32_t sfa_t = tmem_base + (uint32_t)(P4_SF_COL0 + stage * P4_SF_COLS), sfb_t = sfa_t + 16;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            tmem_cp_sf_pair(sfa_t + 4 * k, make_sf_desc(sfa_s + 512 * k));
            tmem_cp_sf_pair(sfb_t + 8 * k, make_sf_desc(sfb_s + 512 * k));             // W rows 0..127 of the tile
            tmem_cp_sf_pair(sfb_t + 8 * k + 4, make_sf_desc(sfb_s + 4 * 512 + 512 * k));  // W rows 128..255
          }
          tc_commit_pair_local(bar_sf + 8 * stage);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  }
  } else {
    // ------------------------------- epilogue warps (both CTAs) -------------------------
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    const int ew = warp - 4;
    const int quad = warp & 3;
    const int half = ew >> 2;
    constexpr int HALF = P4_BN / 2, NCHUNK = HALF / 16;
    const EpiParams& ep = args.ep;
    const int64_t N = args.N;
    const bool has_res = ep.residual != nullptr;
    const float alpha = __ldg(args.a_scale) * __ldg(args.w_scale);
    const uint32_t tempty0 = map_to_cta(bar_tempty, 0);
    EpiBox eb;
    eb.box_s = epi_base + (uint32_t)(ew * P4_NBOX * EPI_BOX_BYTES);
    eb.row_g = epi_gen + ew * P4_NBOX * EPI_BOX_BYTES + lane * 128;
    eb.res_bar = bar_res + 8 * ew;
    eb.res_phase = 0u;
    eb.swz = (uint32_t)(lane & 7);
    uint32_t full_phase = 0u;
    bool ok = true;
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
      int mt, nt;
      pair_tile_coords(tile, args.tiles_m, args.tiles_n, mt, nt);
      const int m_box = mt * 256 + (int)rank * P4_BM + quad * 32;
      const int64_t nbase = (int64_t)nt * P4_BN + half * HALF;
      const int64_t m = (int64_t)m_box + lane;
      const bool row_ok = m < args.M;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(half * HALF);
      const EpiRow row = epi_row_setup(ep, m, row_ok, nbase, N);
      const bool box_rows_in = m_box < args.M;
      const bool use_res = has_res && box_rows_in;
      epi_box_begin<P4_NBOX>(eb, row, use_res, lane, m_box, &tmRes);
      if (!mbar_wait(bar_tfull, full_phase, abort_flag, 4, &g_fp4_status)) { ok = false; break; }
      full_phase ^= 1u;
      tcgen05_fence_after();
      uint32_t acc[NCHUNK][16];
      epi_acc_load<NCHUNK>(taddr, acc);
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty0);  // the accumulator is free again: the leader's barrier collects both CTAs
      if (!epi_box_drain_regs<NCHUNK, true>(eb, row, ep, acc, use_res, box_rows_in, lane, m_box, &tmOut, alpha, abort_flag,
                                            &g_fp4_status)) {
        ok = false;
        break;
      }
    }
    if (lane == 0) bulk_wait_all();
  }

  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();  // nobody leaves while the other CTA may still signal or read it
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// ---- quantiser ----------------------------------------------------------------------------------
__global__ void absmax_bf16_kernel(const __nv_bfloat16* __restrict__ x, int64_t ld, int64_t rows, int K,
                                   float* __restrict__ amax) {
  const int vec_per_row = K >> 3;
  const int64_t total = rows * vec_per_row;
  float m = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / vec_per_row;
    const int c = (int)(i - r * vec_per_row);
    const uint4 v = ldg_nc_u4(x + r * ld + 8 * c);
    float f[8];
    unpack8(v, f);
#pragma unroll
    for (int e = 0; e < 8; ++e) m = fmaxf(m, fabsf(f[e]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) atomicMax(reinterpret_cast<unsigned int*>(amax), __float_as_uint(m));  // m >= 0
}

// one thread per (row, 64-element K tile): 4 blocks of 16 -> 32 bytes of codes + 4 scale bytes
__global__ void quantize_nvfp4_kernel(const __nv_bfloat16* __restrict__ x, int64_t ld, unsigned char* __restrict__ q,
                                      unsigned char* __restrict__ sf, float* __restrict__ scales, int64_t rows, int K,
                                      int ktiles, int ktiles4) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const float amax = fmaxf(scales[0], 1e-30f);
  const float ts = amax / (6.0f * 448.0f);
  if (idx == 0) scales[1] = ts;
  if (idx >= rows * ktiles) return;
  const int64_t r = idx / ktiles;
  const int kt = (int)(idx - r * ktiles);
  const float inv6ts = __frcp_rn(6.0f * ts);
  uint32_t sfw = 0;
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    const int k0 = kt * 64 + b * 16;
    if (k0 >= K) break;
    float f[2][8];
    unpack8(ldg_nc_u4(x + r * ld + k0), f[0]);
    unpack8(ldg_nc_u4(x + r * ld + k0 + 8), f[1]);
    float bm = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) bm = fmaxf(bm, fmaxf(fabsf(f[0][e]), fabsf(f[1][e])));
    const Fp4Block blk = fp4_block_scale(bm, ts, inv6ts);
    sfw |= blk.sf_byte << (8 * b);
    *reinterpret_cast<uint2*>(q + r * (int64_t)(K >> 1) + (k0 >> 1)) = make_uint2(fp4_codes8(f[0], blk.inv), fp4_codes8(f[1], blk.inv));
  }
  const int64_t tile = (r >> 7) * ktiles4 + kt;
  const int rr = (int)(r & 127);
  *reinterpret_cast<uint32_t*>(sf + tile * 512 + (rr & 31) * 16 + (rr >> 5) * 4) = sfw;
}


}  // namespace sana

using namespace sana;

extern "C" int64_t sana_nvfp4_sf_bytes(int64_t rows, int64_t K) {
  if (rows <= 0 || K <= 0) return 0;
  return ceil_div(rows, 128) * ktiles4_of(K) * 512;
}

extern "C" int sana_nvfp4_quantize(const void* x, int64_t ld, void* q, void* sf, float* scales, int64_t rows, int64_t K,
                                   void* stream) {
  SANA_REQUIRE(x && q && sf && scales, "sana_nvfp4_quantize: null pointer");
  SANA_REQUIRE(rows > 0 && K > 0 && K % 32 == 0 && K < (1 << 30), "sana_nvfp4_quantize: K must be a positive multiple of 32");
  SANA_REQUIRE(ld >= K && ld % 8 == 0, "sana_nvfp4_quantize: ld must be >= K and a multiple of 8");
  SANA_REQUIRE(aligned16(x) && aligned16(q) && aligned16(sf) && aligned16(scales), "sana_nvfp4_quantize: alignment");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(scales, 0, 2 * sizeof(float), st);
  if (e != cudaSuccess) return cuda_status(e, "cudaMemsetAsync(scales)");
  e = cudaMemsetAsync(sf, 0, (size_t)sana_nvfp4_sf_bytes(rows, K), st);
  if (e != cudaSuccess) return cuda_status(e, "cudaMemsetAsync(sf)");
  const int64_t vecs = rows * (K / 8);
  int64_t blocks = ceil_div(vecs, 256 * 8);
  if (blocks > 4 * (int64_t)sm_count()) blocks = 4 * (int64_t)sm_count();
  absmax_bf16_kernel<<<(unsigned)blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), ld, rows, (int)K, scales);
  SANA_LAUNCH_CHECK("absmax kernel");
  const int64_t ktiles = ceil_div(K, 64);
  const int64_t total = rows * ktiles;
  SANA_REQUIRE(ceil_div(total, 128) < ((int64_t)1 << 31), "sana_nvfp4_quantize: too large");
  quantize_nvfp4_kernel<<<(unsigned)ceil_div(total, 128), 128, 0, st>>>(
      static_cast<const __nv_bfloat16*>(x), ld, static_cast<unsigned char*>(q), static_cast<unsigned char*>(sf), scales,
      rows, (int)K, (int)ktiles, (int)ktiles4_of(K));
  SANA_LAUNCH_CHECK("quantize kernel");
  return SANA_OK;
}

// Same quantiser with the tensor scale given: scales[0] holds the maximum magnitude to scale for (for example the
// one measured on an earlier call); nothing is measured here.  Values beyond it saturate.
extern "C" int sana_nvfp4_quantize_scaled(const void* x, int64_t ld, void* q, void* sf, float* scales, int64_t rows, int64_t K,
                                          void* stream) {
  SANA_REQUIRE(x && q && sf && scales, "sana_nvfp4_quantize_scaled: null pointer");
  SANA_REQUIRE(rows > 0 && K > 0 && K % 32 == 0 && K < (1 << 30), "sana_nvfp4_quantize_scaled: K must be a positive multiple of 32");
  SANA_REQUIRE(ld >= K && ld % 8 == 0, "sana_nvfp4_quantize_scaled: ld must be >= K and a multiple of 8");
  SANA_REQUIRE(aligned16(x) && aligned16(q) && aligned16(sf) && aligned16(scales), "sana_nvfp4_quantize_scaled: alignment");
  const int64_t ktiles = ceil_div(K, 64);
  const int64_t total = rows * ktiles;
  SANA_REQUIRE(ceil_div(total, 128) < ((int64_t)1 << 31), "sana_nvfp4_quantize_scaled: too large");
  quantize_nvfp4_kernel<<<(unsigned)ceil_div(total, 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), ld, static_cast<unsigned char*>(q), static_cast<unsigned char*>(sf), scales,
      rows, (int)K, (int)ktiles, (int)ktiles4_of(K));
  SANA_LAUNCH_CHECK("quantize kernel");
  return SANA_OK;
}

namespace sana {
// state = n x {amax in use, tensor scale in use, amax seen since the last roll, unused}
__global__ void nvfp4_scale_roll_kernel(float* state, int n, float margin) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float* s = state + 4 * i;
  const float seen = s[2];
  if (seen > 0.f) {
    const float amax = seen * margin;
    s[0] = amax;
    s[1] = fmaxf(amax, 1e-30f) / (6.0f * 448.0f);
    s[2] = 0.f;
  }
}
}  // namespace sana

// Delayed scaling of activations: the kernels that emit FP4 directly (sana_ln_modulate_fp4, sana_la_apply_fp4) and
// sana_nvfp4_quantize_scaled use the tensor scale in state[1] and raise state[2] to the largest magnitude they
// produce (sana_dwconv_glu_amax does the same for its bf16 output); this call adopts what was seen, times `margin`,
// as the scale of the following calls.  `state` holds n records of four floats.
extern "C" int sana_nvfp4_scale_roll(float* state, int64_t n, float margin, void* stream) {
  SANA_REQUIRE(state && n > 0 && n < (1 << 20) && margin > 0.f, "sana_nvfp4_scale_roll: bad arguments");
  nvfp4_scale_roll_kernel<<<(unsigned)ceil_div(n, 64), 64, 0, static_cast<cudaStream_t>(stream)>>>(state, (int)n, margin);
  SANA_LAUNCH_CHECK("nvfp4_scale_roll kernel");
  return SANA_OK;
}

extern "C" int sana_gemm_nvfp4(const void* Aq, const void* sfa, const float* a_scales, const void* Wq, const void* sfw,
                               const float* w_scales, void* out, int64_t ldo, int64_t M, int64_t N, int64_t K,
                               const sana_gemm_epilogue* ep, void* stream) {
  SANA_REQUIRE(Aq && sfa && a_scales && Wq && sfw && w_scales && out, "sana_gemm_nvfp4: null pointer");
  SANA_REQUIRE(M > 0 && N > 0 && K > 0, "sana_gemm_nvfp4: M, N, K must be positive");
  SANA_REQUIRE(K % 32 == 0 && N % 8 == 0 && ldo >= N && ldo % 8 == 0, "sana_gemm_nvfp4: K %% 32, N %% 8, ldo %% 8 required");
  SANA_REQUIRE(M < ((int64_t)1 << 31) && N < ((int64_t)1 << 31) && K < ((int64_t)1 << 30), "sana_gemm_nvfp4: size out of range");
  SANA_REQUIRE(aligned16(Aq) && aligned16(Wq) && aligned16(sfa) && aligned16(sfw) && aligned16(out), "sana_gemm_nvfp4: alignment");
  EpiParams p;
  int rc = check_epilogue(ep, N, &p, "sana_gemm_nvfp4");
  if (rc) return rc;
  SANA_REQUIRE(!p.residual || (aligned16(p.residual) && p.ldr % 8 == 0), "sana_gemm_nvfp4: residual alignment");
  SANA_REQUIRE(!p.bias || aligned16(p.bias), "sana_gemm_nvfp4: bias alignment");
  SANA_REQUIRE(!p.gate_table || (aligned16(p.gate_table) && aligned16(p.gate_t)), "sana_gemm_nvfp4: gate alignment");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // output and residual as 32-row x 64-column boxes (the residual map is a copy when unused)
  CUtensorMap tmA, tmB, tmOut, tmRes;
  rc = make_tmap_2d(&tmOut, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, out, M, N, ldo * 2, 32, EPI_BOX_COLS);
  if (rc) return rc;
  tmRes = tmOut;
  if (p.residual) {
    rc = make_tmap_2d(&tmRes, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.residual, M, N, p.ldr * 2, 32, EPI_BOX_COLS);
    if (rc) return rc;
  }
  const int variant = gemm_variant();
  if (variant == 2 || (variant == 0 && M >= 2048)) {
    // CTA pairs on 256 x 256 tiles
    rc = make_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, Aq, M, K / 2, K / 2, P4_BM, 128);
    if (rc) return rc;
    rc = make_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, Wq, N, K / 2, K / 2, P4_BN / 2, 128);
    if (rc) return rc;
    // the scale buffers as [tiles, 128 words]: a box is the four 512-byte tiles of one K block
    const int64_t kt4 = ktiles4_of(K);
    CUtensorMap tmSFA, tmSFB;
    {
      const uint64_t dims_a[2] = {128, (uint64_t)(ceil_div(M, 128) * kt4)}, dims_b[2] = {128, (uint64_t)(ceil_div(N, 128) * kt4)};
      const uint64_t strides[1] = {512};
      const uint32_t box[2] = {128, 4};
      rc = make_tmap_tiled(&tmSFA, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, sfa, dims_a, strides, box, false);
      if (rc) return rc;
      rc = make_tmap_tiled(&tmSFB, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, sfw, dims_b, strides, box, false);
      if (rc) return rc;
    }
    static OncePerDevice pair_once;
    if (pair_once.first_time()) {
      cudaError_t e = cudaFuncSetAttribute(gemm_nvfp4_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, P4_SMEM_BYTES);
      if (e != cudaSuccess) return cuda_status(e, "cudaFuncSetAttribute(gemm_nvfp4_pair)");
    }
    P4Args a;
    a.out = static_cast<__nv_bfloat16*>(out);
    a.ldo = ldo;
    a.a_scale = a_scales + 1;  // [amax, tensor scale]
    a.w_scale = w_scales + 1;
    a.M = (int)M, a.N = (int)N, a.K = (int)K;
    a.tiles_m = (int)ceil_div(M, 256);
    a.tiles_n = (int)ceil_div(N, P4_BN);
    a.ktiles4 = (int)kt4;
    a.ep = p;
    const int64_t tiles = (int64_t)a.tiles_m * a.tiles_n;
    const int64_t max_clusters = sm_count() / 2;
    const int grid = (int)(2 * (tiles < max_clusters ? tiles : max_clusters));
    gemm_nvfp4_pair_kernel<<<grid, P4_THREADS, P4_SMEM_BYTES, st>>>(tmA, tmB, tmSFA, tmSFB, tmOut, tmRes, a);
    SANA_LAUNCH_CHECK("gemm_nvfp4_pair kernel");
    return SANA_OK;
  }
  rc = make_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, Aq, M, K / 2, K / 2, F4_BM, 128);
  if (rc) return rc;
  rc = make_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, Wq, N, K / 2, K / 2, F4_BN, 128);
  if (rc) return rc;
  static OncePerDevice attr_once;
  if (attr_once.first_time()) {
    cudaError_t e = cudaFuncSetAttribute(gemm_nvfp4_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F4_SMEM_BYTES);
    if (e != cudaSuccess) return cuda_status(e, "cudaFuncSetAttribute(gemm_nvfp4_tc)");
  }
  F4Args a;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.ldo = ldo;
  a.sfa = static_cast<const unsigned char*>(sfa);
  a.sfb = static_cast<const unsigned char*>(sfw);
  a.a_scale = a_scales + 1;  // [amax, tensor scale]
  a.w_scale = w_scales + 1;
  a.M = (int)M, a.N = (int)N, a.K = (int)K;
  a.tiles_m = (int)ceil_div(M, F4_BM);
  a.tiles_n = (int)ceil_div(N, F4_BN);
  a.ktiles4 = (int)ktiles4_of(K);
  a.ep = p;
  const int64_t tiles = (int64_t)a.tiles_m * a.tiles_n;
  const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
  gemm_nvfp4_tc_kernel<<<grid, F4_THREADS, F4_SMEM_BYTES, st>>>(tmA, tmB, tmOut, tmRes, a);
  SANA_LAUNCH_CHECK("gemm_nvfp4_tc kernel");
  return SANA_OK;
}


extern "C" int sana_gemm_nvfp4_take_device_status(int* status_out) {
  if (!status_out) return fail(SANA_ERR_INVALID, "sana_gemm_nvfp4_take_device_status: null pointer");
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_fp4_status, sizeof(int));
  if (e != cudaSuccess) return cuda_status(e, "cudaMemcpyFromSymbol(g_fp4_status)");
  if (v != 0) {
    int zero = 0;
    e = cudaMemcpyToSymbol(g_fp4_status, &zero, sizeof(int));
    if (e != cudaSuccess) return cuda_status(e, "cudaMemcpyToSymbol(g_fp4_status)");
  }
  *status_out = v;
  return SANA_OK;
}
