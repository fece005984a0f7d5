// bf16 projection, CTA-pair variant: two CTAs of a cluster (one SM each) share one 256 x BN
// output tile.  Each CTA loads its own 128 rows of A and HALF of the W tile (BN/2 rows) into
// its shared memory (plain TMA loads, no multicast); the pair's leader (cluster rank 0)
// issues tcgen05.mma.cta_group::2 (M = 256), which reads both halves of W and writes each
// CTA's 128 accumulator rows into that CTA's tensor memory.  Per SM this moves 30 KiB per K
// block through shared memory instead of 44 KiB for the same math, which is what keeps the
// tensor pipe fed.  Pipeline and bounded waits are those of the single-CTA kernel; the epilogue
// goes through shared-memory boxes and bulk-tensor copies (see the epilogue warps below).
//
// Barriers: full[s] lives in the leader and counts the bytes of BOTH CTAs' loads; empty[s]
// and tfull[a] live in both CTAs and are signalled by the leader's tcgen05.commit with a
// two-CTA arrive mask; tempty[a] lives in the leader and collects the 16 epilogue warps of
// the pair (the peer's warps arrive remotely).
#include "tc_common.cuh"

namespace sana {

__device__ int g_gemm2_status = 0;  // soft-error word of this kernel's bounded waits

constexpr int T2_BM = 128;                      // rows per CTA (256 per pair)
constexpr int T2_BK = 64;
constexpr int T2_A_BYTES = T2_BM * T2_BK * 2;   // 16 KiB
constexpr int T2_EPI_WARPS = 8;
constexpr int T2_THREADS = 64 + 32 * T2_EPI_WARPS;
constexpr int T2_SMEM_LIMIT = 232448;
constexpr int T2_CTRL_BYTES = 256;

template <int BN>
struct T2Cfg {
  static constexpr int BH = BN / 2;                       // W rows held by each CTA
  static constexpr int B_BYTES = BH * T2_BK * 2;
  static constexpr int STAGE_BYTES = T2_A_BYTES + B_BYTES;
  static constexpr int HALF = BN / 2;                     // columns per epilogue warp
  static constexpr int NCHUNK = HALF / 16;
  static constexpr int NBOX = HALF / EPI_BOX_COLS;         // staging boxes per epilogue warp
  static constexpr int EPI_BYTES = T2_EPI_WARPS * NBOX * EPI_BOX_BYTES;
  static constexpr int MAX_STAGES = (T2_SMEM_LIMIT - T2_CTRL_BYTES - EPI_BYTES) / STAGE_BYTES;
  static constexpr int STAGES = MAX_STAGES > 8 ? 8 : MAX_STAGES;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + T2_CTRL_BYTES;
  static constexpr int TMEM_COLS = (2 * BN <= 256) ? 256 : 512;
  // D=f32, A=B=bf16, K-major, N>>3 at bit 17, M=256 (>>4) at bit 24
  static constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                                    ((uint32_t)(256 >> 4) << 24);
  static_assert(BN == 128 || BN == 256, "the staged epilogue needs column halves that are whole 64-column boxes");
  static_assert(STAGE_BYTES % 1024 == 0, "stage bases must stay 1024-byte aligned");
  static_assert(STAGES >= 4, "too few pipeline stages");
  static_assert(16 * STAGES + 40 + 8 * T2_EPI_WARPS <= T2_CTRL_BYTES, "control block too small");
};

struct T2Args {
  __nv_bfloat16* out;
  int64_t ldo;
  int M, N, K;
  int tiles_m, tiles_n;  // tiles_m counts 256-row pair tiles
  EpiParams ep;
};

template <int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(T2_THREADS, 1)
gemm_bf16_tc2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const __grid_constant__ CUtensorMap tmOut, const __grid_constant__ CUtensorMap tmRes,
                     const T2Args args) {
  using Cfg = T2Cfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t tiles_base = smem_u32(smem_raw);
  const uint32_t epi_base = tiles_base + STAGES * Cfg::STAGE_BYTES;  // staging boxes of the epilogue warps
  unsigned char* epi_gen = smem_raw + STAGES * Cfg::STAGE_BYTES;
  const uint32_t ctrl = epi_base + Cfg::EPI_BYTES;
  unsigned char* ctrl_gen = epi_gen + Cfg::EPI_BYTES;
  // control layout: full[STAGES] | empty[STAGES] | tfull[2] | tempty[2] | tmem ptr | abort | res[EPI_WARPS]
  const uint32_t bar_full = ctrl, bar_empty = ctrl + 8 * STAGES;
  const uint32_t bar_tfull = ctrl + 16 * STAGES, bar_tempty = bar_tfull + 16;
  const uint32_t bar_res = ctrl + 16 * STAGES + 40;
  volatile uint32_t* tmem_ptr_slot = reinterpret_cast<volatile uint32_t*>(ctrl_gen + 16 * STAGES + 32);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(ctrl_gen + 16 * STAGES + 36);

  // the dynamic shared window starts at the same offset in every CTA, so this is cluster-uniform
  if ((tiles_base & 1023u) != 0u) {
    if (threadIdx.x == 0) atomicExch(&g_gemm2_status, 9);
    return;
  }

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  const int num_tiles = args.tiles_m * args.tiles_n;
  const int kblocks = (args.K + T2_BK - 1) / T2_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, 2 * T2_EPI_WARPS);
    }
    for (int w = 0; w < T2_EPI_WARPS; ++w) mbar_init(bar_res + 8 * w, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmA) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmOut) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmRes) : "memory");
  }
  if (warp == 1) {  // the same warp of both CTAs allocates collectively
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ctrl + 16 * STAGES + 32),
                 "r"((uint32_t)Cfg::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything signals them
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_ptr_slot;

  if (warp == 0) {
    // ------------------------------- TMA producer (both CTAs) ---------------------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      const uint32_t full0 = map_to_cta(bar_full, 0);  // the leader's full barriers, cluster address
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        int tm, tn;
        pair_tile_coords(tile, args.tiles_m, args.tiles_n, tm, tn);
        const int m0 = tm * (2 * T2_BM) + (int)rank * T2_BM;
        // a ragged last tile column is computed at its own width (a multiple of 32): each CTA then holds half of
        // THAT many W rows, not half of BN
        const int nt0 = tn * BN;
        const int n_this = min(BN, ((args.N - nt0) + 31) & ~31);
        const int n0 = nt0 + (int)rank * (n_this >> 1);
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, 1, &g_gemm2_status)) { ok = false; break; }
          const uint32_t sa = tiles_base + stage * Cfg::STAGE_BYTES;
          if (leader) mbar_expect_tx(bar_full + 8 * stage, 2 * Cfg::STAGE_BYTES);
          tma_load_2d_pair(sa, &tmA, full0 + 8 * stage, kb * T2_BK, m0);
          tma_load_2d_pair(sa + T2_A_BYTES, &tmB, full0 + 8 * stage, kb * T2_BK, n0);
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
      uint32_t stage = 0, phase = 0;
      uint32_t acc_phase = 0u;
      bool ok = true;
      int it = 0;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters, ++it) {
        const int a = it & 1;
        if (!mbar_wait(bar_tempty + 8 * a, ((acc_phase >> a) & 1u) ^ 1u, abort_flag, 2, &g_gemm2_status)) { ok = false; break; }
        acc_phase ^= 1u << a;
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(a * BN);
        int tm, tn;
        pair_tile_coords(tile, args.tiles_m, args.tiles_n, tm, tn);
        const int n_this = min(BN, ((args.N - tn * BN) + 31) & ~31);
        // same descriptor with this tile's N (>> 3 at bit 17)
        const uint32_t idesc = (Cfg::IDESC & ~(0x3Fu << 17)) | ((uint32_t)(n_this >> 3) << 17);
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, 3, &g_gemm2_status)) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t sa = tiles_base + stage * Cfg::STAGE_BYTES;
          const uint64_t adesc = make_smem_desc(sa), bdesc = make_smem_desc(sa + T2_A_BYTES);
#pragma unroll
          for (int k = 0; k < T2_BK / 16; ++k)
            umma_bf16_pair(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit_pair(bar_empty + 8 * stage);  // frees this stage in both CTAs
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit_pair(bar_tfull + 8 * a);  // accumulator complete, both CTAs
      }
    }
  } else {
    // ------------------------------- epilogue warps (both CTAs) -------------------------
    // staged epilogue (tc_common.cuh): a warp owns 32 rows x one column half = NBOX boxes
    const int ew = warp - 2;
    const int quad = warp & 3;
    const int half = ew >> 2;
    const EpiParams& ep = args.ep;
    const int64_t N = args.N;
    const bool has_res = ep.residual != nullptr;
    const uint32_t tempty0 = map_to_cta(bar_tempty, 0);
    EpiBox eb;
    eb.box_s = epi_base + (uint32_t)(ew * Cfg::NBOX * EPI_BOX_BYTES);
    eb.row_g = epi_gen + ew * Cfg::NBOX * EPI_BOX_BYTES + lane * 128;
    eb.res_bar = bar_res + 8 * ew;
    eb.res_phase = 0u;
    eb.swz = (uint32_t)(lane & 7);
    uint32_t full_phase = 0u;
    bool ok = true;
    int it = 0;
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters, ++it) {
      const int a = it & 1;
      int tm, tn;
      pair_tile_coords(tile, args.tiles_m, args.tiles_n, tm, tn);
      const int m_box = tm * (2 * T2_BM) + (int)rank * T2_BM + quad * 32;
      const int64_t nbase = (int64_t)tn * BN + half * Cfg::HALF;
      const int64_t m = (int64_t)m_box + lane;
      const bool row_ok = m < args.M;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(a * BN + half * Cfg::HALF);
      const EpiRow row = epi_row_setup(ep, m, row_ok, nbase, N);
      const bool box_rows_in = m_box < args.M;  // otherwise the whole box lies below the matrix: no copies
      const bool use_res = has_res && box_rows_in;
      epi_box_begin<Cfg::NBOX>(eb, row, use_res, lane, m_box, &tmRes);
      EpiStep st[2];
      epi_fetch(row, st[0], 0);  // operands that do not depend on the accumulator: requested before the wait
      if (!mbar_wait(bar_tfull + 8 * a, (full_phase >> a) & 1u, abort_flag, 4, &g_gemm2_status)) { ok = false; break; }
      full_phase ^= 1u << a;
      tcgen05_fence_after();
      if (!epi_box_drain<Cfg::NCHUNK, false>(eb, row, ep, taddr, st, use_res, box_rows_in, lane, m_box, &tmOut, 1.0f,
                                             abort_flag, &g_gemm2_status)) {
        ok = false;
        break;
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty0 + 8 * a);  // the leader's barrier collects both CTAs
    }
    if (lane == 0) bulk_wait_all();  // the boxes stay valid until the last stores have drained
  }

  // ------------------------------- teardown ---------------------------------------------
  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();  // nobody leaves while the other CTA may still signal or read it
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::TMEM_COLS)
                 : "memory");
  }
}

// ---- host side ------------------------------------------------------------------------------
template <int BN>
static int launch_pair_bn(const void* A, int64_t lda, const void* Wt, int64_t ldw, int64_t M, int64_t N, int64_t K,
                          T2Args& args, cudaStream_t st) {
  using Cfg = T2Cfg<BN>;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, M, K, lda * 2, T2_BM, T2_BK);
  if (rc) return rc;
  rc = make_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Wt, N, K, ldw * 2, Cfg::BH, T2_BK);
  if (rc) return rc;
  // output and residual as 32-row x 64-column boxes (the residual map is a copy when unused)
  CUtensorMap tmOut, tmRes;
  rc = make_tmap_2d(&tmOut, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, args.out, M, N, args.ldo * 2, 32, EPI_BOX_COLS);
  if (rc) return rc;
  if (args.ep.residual) {
    rc = make_tmap_2d(&tmRes, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, args.ep.residual, M, N, args.ep.ldr * 2, 32, EPI_BOX_COLS);
    if (rc) return rc;
  } else {
    tmRes = tmOut;
  }
  static OncePerDevice attr_once;
  if (attr_once.first_time()) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_tc2_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return cuda_status(e, "cudaFuncSetAttribute(gemm_bf16_tc2)");
  }
  args.tiles_n = (int)ceil_div(N, BN);
  const int64_t tiles = (int64_t)args.tiles_m * args.tiles_n;
  const int64_t max_clusters = sm_count() / 2;
  const int grid = (int)(2 * (tiles < max_clusters ? tiles : max_clusters));
  gemm_bf16_tc2_kernel<BN><<<grid, T2_THREADS, Cfg::SMEM_BYTES, st>>>(tmA, tmB, tmOut, tmRes, args);
  SANA_LAUNCH_CHECK("gemm_bf16_tc2 kernel");
  return SANA_OK;
}

int gemm_tc2_launch(const void* A, int64_t lda, const void* Wt, int64_t ldw, void* out, int64_t ldo, int64_t M,
                    int64_t N, int64_t K, const EpiParams& ep, cudaStream_t st) {
  T2Args args;
  args.out = static_cast<__nv_bfloat16*>(out);
  args.ldo = ldo;
  args.M = (int)M, args.N = (int)N, args.K = (int)K;
  args.tiles_m = (int)ceil_div(M, 2 * T2_BM);
  args.tiles_n = 0;
  args.ep = ep;
  // tile width: minimise (waves over the CTA pairs) x BN; the narrow tile carries a 12 % handicap
  // because, per column, narrower tiles measured that much slower than 256 (256 was 4-10 % faster
  // end to end on N = 2240 / 6720 / 11200 even where it leaves a ragged last tile)
  const int cands[2] = {256, 128};
  const int64_t clusters = sm_count() / 2;
  int best = 128;
  int64_t best_cost = -1;
  for (int bn : cands) {
    const int64_t cost = ceil_div((int64_t)args.tiles_m * ceil_div(N, bn), clusters) * bn * (bn == 256 ? 100 : 112);
    if (best_cost < 0 || cost < best_cost) best_cost = cost, best = bn;
  }
  switch (best) {
    case 256: return launch_pair_bn<256>(A, lda, Wt, ldw, M, N, K, args, st);
    default: return launch_pair_bn<128>(A, lda, Wt, ldw, M, N, K, args, st);
  }
}

int gemm_tc2_take_status(int* v) {
  cudaError_t e = cudaMemcpyFromSymbol(v, g_gemm2_status, sizeof(int));
  if (e != cudaSuccess) return cuda_status(e, "cudaMemcpyFromSymbol(g_gemm2_status)");
  if (*v != 0) {
    int zero = 0;
    e = cudaMemcpyToSymbol(g_gemm2_status, &zero, sizeof(int));
    if (e != cudaSuccess) return cuda_status(e, "cudaMemcpyToSymbol(g_gemm2_status)");
  }
  return SANA_OK;
}

}  // namespace sana
