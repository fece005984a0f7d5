// bf16 projection on the 5th-generation tensor cores: out = epilogue(A[M,K] @ Wt[N,K]^T).
//
// Persistent, warp-specialised kernel, one CTA per SM, 128 x BN output tiles:
//   warp 0 (one lane)  TMA producer: 128x64 A tile + BNx64 W tile per K block into a ring of
//                      128-byte-swizzled shared-memory stages (no multicast; out-of-range
//                      rows / K tail are zero-filled by the TMA unit)
//   warp 1 (one lane)  issues tcgen05.mma (M=128, N=BN, K=16 per instruction), accumulating
//                      in tensor memory; two accumulator buffers so the epilogue of tile i
//                      overlaps the MMAs of tile i+1
//   warps 2..9         epilogue: two warps per TMEM lane quadrant (left / right half of the
//                      tile), tcgen05.ld of 16 columns per step with the next step's
//                      accumulator, bias, gate and residual operands already in flight;
//                      bias / activation / adaLN gate / residual in fp32, 16-byte stores
// Every wait is bounded: after ~2 s a role records a code in g_gemm_status, raises the
// CTA-wide abort flag and all roles fall through to the common teardown (TMEM is freed).
#include <mutex>

#include <string.h>

#include <mutex>
#include <unordered_map>

#include "tc_common.cuh"

namespace sana {

__device__ int g_gemm_status = 0;

constexpr int TC_BM = 128;
constexpr int TC_BK = 64;                       // 64 bf16 = one 128-byte swizzle row
constexpr int TC_A_BYTES = TC_BM * TC_BK * 2;   // 16 KiB
constexpr int TC_EPI_WARPS = 8;                 // two warps per TMEM lane quadrant (left / right half of the tile)
constexpr int TC_THREADS = 64 + 32 * TC_EPI_WARPS;
constexpr int TC_SMEM_LIMIT = 232448;           // 227 KiB opt-in maximum per CTA
constexpr int TC_CTRL_BYTES = 256;              // barriers + tmem pointer + abort flag

template <int BN>
struct TcCfg {
  static constexpr int B_BYTES = BN * TC_BK * 2;
  static constexpr int STAGE_BYTES = TC_A_BYTES + B_BYTES;
  static constexpr int HALF = BN / 2;              // columns per epilogue warp
  static constexpr int NCHUNK = HALF / 16;         // 16-column steps per epilogue warp
  static constexpr int NBOX = HALF / EPI_BOX_COLS;  // staging boxes per epilogue warp (tc_common.cuh)
  static constexpr int EPI_BYTES = TC_EPI_WARPS * NBOX * EPI_BOX_BYTES;
  static constexpr int MAX_STAGES = (TC_SMEM_LIMIT - TC_CTRL_BYTES - EPI_BYTES) / STAGE_BYTES;
  static constexpr int STAGES = MAX_STAGES > 6 ? 6 : MAX_STAGES;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + TC_CTRL_BYTES;
  static constexpr int TMEM_COLS = (2 * BN <= 256) ? 256 : 512;
  // instruction descriptor: D=f32 (bit 4), A=B=bf16 (bits 7, 10), both K-major, N>>3 at 17, M>>4 at 24
  static constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                                    ((uint32_t)(TC_BM >> 4) << 24);
  static_assert(BN == 128 || BN == 256, "the staged epilogue needs column halves that are whole 64-column boxes");
  static_assert(STAGES >= 3, "not enough shared memory for the ring");
  static_assert(16 * STAGES + 40 + 8 * TC_EPI_WARPS <= TC_CTRL_BYTES, "control block too small");
};

struct TcArgs {
  __nv_bfloat16* out;
  int64_t ldo;
  int M, N, K;
  int tiles_m, tiles_n;
  EpiParams ep;
};

template <int BN>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_bf16_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmOut, const __grid_constant__ CUtensorMap tmRes,
                    const TcArgs args) {
  using Cfg = TcCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t tiles_base = smem_u32(smem_raw);                // swizzled tiles need 1024-byte alignment
  const uint32_t epi_base = tiles_base + STAGES * Cfg::STAGE_BYTES;  // staging boxes of the epilogue warps
  unsigned char* epi_gen = smem_raw + STAGES * Cfg::STAGE_BYTES;
  const uint32_t ctrl = epi_base + Cfg::EPI_BYTES;                   // control block after them
  unsigned char* ctrl_gen = epi_gen + Cfg::EPI_BYTES;
  // control layout: full[STAGES] | empty[STAGES] | tfull[2] | tempty[2] | tmem ptr | abort | res[EPI_WARPS]
  const uint32_t bar_full = ctrl, bar_empty = ctrl + 8 * STAGES;
  const uint32_t bar_tfull = ctrl + 16 * STAGES, bar_tempty = bar_tfull + 16;
  const uint32_t bar_res = ctrl + 16 * STAGES + 40;
  volatile uint32_t* tmem_ptr_slot = reinterpret_cast<volatile uint32_t*>(ctrl_gen + 16 * STAGES + 32);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(ctrl_gen + 16 * STAGES + 36);

  if ((tiles_base & 1023u) != 0u) {  // uniform over the CTA: nothing has been set up yet
    if (threadIdx.x == 0) atomicExch(&g_gemm_status, 9);
    return;
  }

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = args.tiles_m * args.tiles_n;
  const int kblocks = (args.K + TC_BK - 1) / TC_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, TC_EPI_WARPS);
    }
    for (int w = 0; w < TC_EPI_WARPS; ++w) mbar_init(bar_res + 8 * w, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmA) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmOut) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmRes) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ctrl + 16 * STAGES + 32),
                 "r"((uint32_t)Cfg::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_ptr_slot;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile / args.tiles_n) * TC_BM, n0 = (tile % args.tiles_n) * BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, 1, &g_gemm_status)) { ok = false; break; }
          const uint32_t sa = tiles_base + stage * Cfg::STAGE_BYTES;
          mbar_expect_tx(bar_full + 8 * stage, Cfg::STAGE_BYTES);
          tma_load_2d(sa, &tmA, bar_full + 8 * stage, kb * TC_BK, m0);
          tma_load_2d(sa + TC_A_BYTES, &tmB, bar_full + 8 * stage, kb * TC_BK, n0);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // give copies already in flight time to land before the CTA tears down
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ---------------------------------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      uint32_t acc_phase = 0u;  // bit a = phase of accumulator buffer a
      bool ok = true;
      int it = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
        const int a = it & 1;
        if (!mbar_wait(bar_tempty + 8 * a, ((acc_phase >> a) & 1u) ^ 1u, abort_flag, 2, &g_gemm_status)) { ok = false; break; }
        acc_phase ^= 1u << a;
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(a * BN);
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, 3, &g_gemm_status)) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t sa = tiles_base + stage * Cfg::STAGE_BYTES;
          const uint64_t adesc = make_smem_desc(sa), bdesc = make_smem_desc(sa + TC_A_BYTES);
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k) {
            // +32 bytes per K=16 step inside the 128-byte swizzle row (address field is >>4)
            umma_bf16(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), Cfg::IDESC, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(bar_empty + 8 * stage);  // stage reusable once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(bar_tfull + 8 * a);  // accumulator complete
      }
    }
  } else {
    // ------------------------------- epilogue warps -----------------------------------
    // warp w reads TMEM lanes 32*(w%4)..+31 (hardware rule) and the left or right half of the
    // tile's columns; 16 columns per step, operands of step c+1 in flight while step c is
    // computed and stored.
    const int ew = warp - 2;
    const int quad = warp & 3;
    const int half = ew >> 2;
    const EpiParams& ep = args.ep;
    const int64_t N = args.N;
    const bool has_res = ep.residual != nullptr;
    EpiBox eb;
    eb.box_s = epi_base + (uint32_t)(ew * Cfg::NBOX * EPI_BOX_BYTES);
    eb.row_g = epi_gen + ew * Cfg::NBOX * EPI_BOX_BYTES + lane * 128;
    eb.res_bar = bar_res + 8 * ew;
    eb.res_phase = 0u;
    eb.swz = (uint32_t)(lane & 7);
    uint32_t full_phase = 0u;  // bit a = phase of accumulator buffer a
    bool ok = true;
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
      const int a = it & 1;
      const int m_box = (tile / args.tiles_n) * TC_BM + quad * 32;
      const int64_t nbase = (int64_t)(tile % args.tiles_n) * BN + half * Cfg::HALF;
      const int64_t m = (int64_t)m_box + lane;
      const bool row_ok = m < args.M;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(a * BN + half * Cfg::HALF);
      const EpiRow row = epi_row_setup(ep, m, row_ok, nbase, N);
      const bool box_rows_in = m_box < args.M;  // otherwise the whole box lies below the matrix: no copies
      const bool use_res = has_res && box_rows_in;
      epi_box_begin<Cfg::NBOX>(eb, row, use_res, lane, m_box, &tmRes);
      EpiStep st[2];
      epi_fetch(row, st[0], 0);  // operands that do not depend on the accumulator: requested before the wait
      if (!mbar_wait(bar_tfull + 8 * a, (full_phase >> a) & 1u, abort_flag, 4, &g_gemm_status)) { ok = false; break; }
      full_phase ^= 1u << a;
      tcgen05_fence_after();
      if (!epi_box_drain<Cfg::NCHUNK, false>(eb, row, ep, taddr, st, use_res, box_rows_in, lane, m_box, &tmOut, 1.0f,
                                             abort_flag, &g_gemm_status)) {
        ok = false;
        break;
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + 8 * a);
    }
    if (lane == 0) bulk_wait_all();  // the boxes stay valid until the last stores have drained
  }

  // ------------------------------- teardown ---------------------------------------------
  __syncwarp();  // single-lane roles rejoin their warp before the CTA-wide barrier
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::TMEM_COLS)
                 : "memory");
  }
}

// ---- host side ------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// Encoded maps are kept in a process-wide cache keyed by everything that goes into them (data type,
// base address, extents, strides, box, swizzle): a forward pass asks for the same few dozen maps on
// every step, and an encode call costs about as much as a small kernel launch.  A map depends only
// on its key, not on the contents of memory or on the device, so a stale entry cannot exist; the
// cache is emptied when it reaches its size limit.
struct TmapKey {
  uint64_t w[14];
  bool operator==(const TmapKey& o) const { return memcmp(w, o.w, sizeof(w)) == 0; }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    uint64_t h = 1469598103934665603ull;
    for (uint64_t v : k.w) h = (h ^ v) * 1099511628211ull;
    return (size_t)h;
  }
};
static std::mutex g_tmap_mutex;
static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> g_tmap_cache;
constexpr size_t TMAP_CACHE_LIMIT = 8192;

int make_tmap_tiled(CUtensorMap* tm, CUtensorMapDataType dtype, int rank, const void* base, const uint64_t* dims,
                    const uint64_t* strides_bytes, const uint32_t* box, bool swizzle128) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(SANA_ERR_DRIVER, "cuTensorMapEncodeTiled is not available from the driver");
  if (rank < 1 || rank > 5) return fail(SANA_ERR_INVALID, "tensor map rank %d out of range", rank);
  TmapKey key = {};
  key.w[0] = (uint64_t)dtype | ((uint64_t)rank << 8) | ((uint64_t)(swizzle128 ? 1 : 0) << 16);
  key.w[1] = (uint64_t)reinterpret_cast<uintptr_t>(base);
  for (int i = 0; i < rank; ++i) key.w[2 + i] = dims[i];
  for (int i = 0; i + 1 < rank; ++i) key.w[7 + i] = strides_bytes[i];
  for (int i = 0; i < rank; ++i) key.w[11 + i / 2] |= (uint64_t)box[i] << (32 * (i & 1));
  {
    std::lock_guard<std::mutex> lock(g_tmap_mutex);
    auto it = g_tmap_cache.find(key);
    if (it != g_tmap_cache.end()) {
      *tm = it->second;
      return SANA_OK;
    }
  }
  cuuint64_t d[5], s[5];
  cuuint32_t b[5], estr[5];
  for (int i = 0; i < rank; ++i) d[i] = dims[i], b[i] = box[i], estr[i] = 1;
  for (int i = 0; i + 1 < rank; ++i) s[i] = strides_bytes[i];
  CUresult r = fn(tm, dtype, (cuuint32_t)rank, const_cast<void*>(base), d, s, b, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(SANA_ERR_DRIVER, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  std::lock_guard<std::mutex> lock(g_tmap_mutex);
  if (g_tmap_cache.size() >= TMAP_CACHE_LIMIT) g_tmap_cache.clear();
  g_tmap_cache.emplace(key, *tm);
  return SANA_OK;
}

int make_tmap_2d(CUtensorMap* tm, CUtensorMapDataType dtype, int elem_bytes, const void* base, int64_t rows,
                 int64_t cols, int64_t ld_bytes, int box_rows, int box_cols) {
  (void)elem_bytes;
  const uint64_t dims[2] = {(uint64_t)cols, (uint64_t)rows};
  const uint64_t strides[1] = {(uint64_t)ld_bytes};
  const uint32_t box[2] = {(uint32_t)box_cols, (uint32_t)box_rows};
  return make_tmap_tiled(tm, dtype, 2, base, dims, strides, box, true);
}

// [rows, cols] bf16 matrix, row stride ld elements; box = box_rows x 64 columns.
static int make_tmap(CUtensorMap* tm, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
  return make_tmap_2d(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, rows, cols, ld * 2, box_rows, TC_BK);
}

template <int BN>
static int launch_bn(const CUtensorMap& tmA, const void* Wt, int64_t ldw, int64_t N, int64_t K, TcArgs& args,
                     cudaStream_t st) {
  using Cfg = TcCfg<BN>;
  CUtensorMap tmB, tmOut, tmRes;
  int rc = make_tmap(&tmB, Wt, N, K, ldw, BN);
  if (rc) return rc;
  // output and residual as 32-row x 64-column boxes (the residual map is a copy when unused)
  rc = make_tmap(&tmOut, args.out, args.M, N, args.ldo, 32);
  if (rc) return rc;
  tmRes = tmOut;
  if (args.ep.residual) {
    rc = make_tmap(&tmRes, args.ep.residual, args.M, N, args.ep.ldr, 32);
    if (rc) return rc;
  }
  static OncePerDevice attr_once;
  if (attr_once.first_time()) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return cuda_status(e, "cudaFuncSetAttribute(gemm_bf16_tc)");
  }
  args.tiles_n = (int)ceil_div(N, BN);
  const int64_t tiles = (int64_t)args.tiles_m * args.tiles_n;
  const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
  gemm_bf16_tc_kernel<BN><<<grid, TC_THREADS, Cfg::SMEM_BYTES, st>>>(tmA, tmB, tmOut, tmRes, args);
  SANA_LAUNCH_CHECK("gemm_bf16_tc kernel");
  return SANA_OK;
}

// Tile width: minimise (waves over the SMs) x BN, i.e. padded work including the last partial wave.
static int pick_bn(int64_t M, int64_t N) {
  const int cands[2] = {256, 128};
  const int64_t sms = sm_count();
  const int64_t tm = ceil_div(M, TC_BM);
  int best = 128;
  int64_t best_cost = -1;
  for (int bn : cands) {
    const int64_t tiles = tm * ceil_div(N, bn);
    const int64_t cost = ceil_div(tiles, sms) * bn;
    if (best_cost < 0 || cost < best_cost) best_cost = cost, best = bn;
  }
  return best;
}

int gemm_tc2_launch(const void* A, int64_t lda, const void* Wt, int64_t ldw, void* out, int64_t ldo, int64_t M,
                    int64_t N, int64_t K, const EpiParams& ep, cudaStream_t st);
int gemm_tc2_take_status(int* v);

// 0 = choose per problem, 1 = always the single-CTA kernel, 2 = always the CTA-pair kernel
static int g_gemm_variant = 0;
int gemm_variant() { return g_gemm_variant; }

int gemm_tc_launch(const void* A, int64_t lda, const void* Wt, int64_t ldw, void* out, int64_t ldo, int64_t M,
                   int64_t N, int64_t K, const EpiParams& ep, cudaStream_t st) {
  SANA_REQUIRE(aligned16(A) && aligned16(Wt) && aligned16(out), "sana_gemm: pointers must be 16-byte aligned");
  SANA_REQUIRE(lda % 8 == 0 && ldw % 8 == 0 && ldo % 8 == 0, "sana_gemm: row strides must be multiples of 8 (bf16)");
  SANA_REQUIRE(N % 8 == 0, "sana_gemm: N must be a multiple of 8 (bf16)");
  SANA_REQUIRE(!ep.residual || (aligned16(ep.residual) && ep.ldr % 8 == 0), "sana_gemm: residual alignment");
  SANA_REQUIRE(!ep.bias || aligned16(ep.bias), "sana_gemm: bias alignment");
  SANA_REQUIRE(!ep.gate_table || (aligned16(ep.gate_table) && aligned16(ep.gate_t)), "sana_gemm: gate alignment");
  // CTA pairs pay off once there are enough 256-row tiles to fill the device
  const bool pair = g_gemm_variant == 2 || (g_gemm_variant == 0 && M >= 2048);
  if (pair) return gemm_tc2_launch(A, lda, Wt, ldw, out, ldo, M, N, K, ep, st);
  CUtensorMap tmA;
  int rc = make_tmap(&tmA, A, M, K, lda, TC_BM);
  if (rc) return rc;
  TcArgs args;
  args.out = static_cast<__nv_bfloat16*>(out);
  args.ldo = ldo;
  args.M = (int)M, args.N = (int)N, args.K = (int)K;
  args.tiles_m = (int)ceil_div(M, TC_BM);
  args.tiles_n = 0;
  args.ep = ep;
  switch (pick_bn(M, N)) {
    case 256: return launch_bn<256>(tmA, Wt, ldw, N, K, args, st);
    default: return launch_bn<128>(tmA, Wt, ldw, N, K, args, st);
  }
}

}  // namespace sana

extern "C" int sana_gemm_take_device_status(int* status_out) {
  if (!status_out) return sana::fail(SANA_ERR_INVALID, "sana_gemm_take_device_status: null pointer");
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, sana::g_gemm_status, sizeof(int));
  if (e != cudaSuccess) return sana::cuda_status(e, "cudaMemcpyFromSymbol(g_gemm_status)");
  if (v != 0) {
    int zero = 0;
    e = cudaMemcpyToSymbol(sana::g_gemm_status, &zero, sizeof(int));
    if (e != cudaSuccess) return sana::cuda_status(e, "cudaMemcpyToSymbol(g_gemm_status)");
  }
  int v2 = 0;
  int rc = sana::gemm_tc2_take_status(&v2);
  if (rc) return rc;
  *status_out = v != 0 ? v : (v2 != 0 ? 100 + v2 : 0);  // 1xx = recorded by the CTA-pair kernel
  return SANA_OK;
}

extern "C" int sana_gemm_set_variant(int variant) {
  if (variant < 0 || variant > 2) return sana::fail(SANA_ERR_INVALID, "sana_gemm_set_variant: 0, 1 or 2");
  sana::g_gemm_variant = variant;
  return SANA_OK;
}
