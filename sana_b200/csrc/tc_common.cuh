// PTX wrappers shared by the tensor-core projection kernels (bf16 and NVFP4): mbarriers with
// bounded waits, TMA loads, tcgen05 MMA / commit / TMEM loads, shared-memory descriptors.
#pragma once
#include <cuda.h>

#include "epilogue.cuh"

namespace sana {

// ---- PTX wrappers ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// One poll of a barrier phase.  The last operand is the time the hardware may keep the thread suspended
// before the poll returns "not yet": without it a waiting warp comes back every few dozen cycles, and the
// eight epilogue warps of a GEMM CTA, which wait for most of a tile's duration, then spend enough issue slots
// and power on polling to cost 4 % of the power-capped GEMM rate (1 219 -> 1 265 TFLOP/s over the four
// projection shapes run for two seconds).
#ifndef SANA_WAIT_HINT_NS
#define SANA_WAIT_HINT_NS 1000
#endif
#define SANA_STR2(x) #x
#define SANA_STR(x) SANA_STR2(x)
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, " SANA_STR(SANA_WAIT_HINT_NS) ";\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// The same poll without the hint, for warps that are fed row by row and should be back at once (depthwise kernel).
__device__ __forceinline__ bool mbar_try_wait_poll(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

constexpr long long TC_WAIT_LIMIT_CYCLES = 4000000000LL;  // ~2 s at 2 GHz

// Bounded wait.  Returns false (and raises the abort flag) on time-out or when another role
// already aborted; `status_word` is the global soft-error word that records the code.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code,
                                          int* status_word) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 255u) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > TC_WAIT_LIMIT_CYCLES) {
        *abort_flag = code;
        atomicExch(status_word, code);
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* tmap, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives on the mbarrier once all previously issued MMAs of this thread have completed
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major, 128-byte-swizzled operand tile: rows of 128 bytes, 8-row groups 1024 bytes apart.
// bits 0-13 address>>4, 16-29 leading offset (1, unused for swizzled K-major), 32-45 stride
// offset (1024>>4), 46-47 descriptor version 1, 61-63 layout 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  const uint32_t lo = ((saddr >> 4) & 0x3FFFu) | (1u << 16);
  const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
  return ((uint64_t)hi << 32) | lo;
}

__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ float fast_silu(float x) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-1.4426950408889634f * x));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return x * r;
}

// ---- fused epilogue: per-row set-up and the small per-column operands ------------------------
// An epilogue warp owns 32 accumulator rows (its TMEM lane quadrant) and NCHUNK steps of 16
// columns.  Per step a lane needs 16 accumulator words plus 32 bytes each of bias, gate table
// and gate timestep vector (the same for every row: broadcast loads, issued one step ahead of
// their use); the residual and the output go through the staged boxes below.
struct EpiStep {
  uint32_t acc[16];
  uint4 bias[2], gtab[2], gt[2];
};

struct EpiRow {
  const __nv_bfloat16 *bias, *grow, *gtrow;
  int64_t nbase, N;
};

// m = this lane's row, row_ok = it lies inside the matrix (else sample 0's gate vector is read)
__device__ __forceinline__ EpiRow epi_row_setup(const EpiParams& ep, int64_t m, bool row_ok, int64_t nbase, int64_t N) {
  EpiRow r;
  r.bias = static_cast<const __nv_bfloat16*>(ep.bias);
  const __nv_bfloat16* gtab = static_cast<const __nv_bfloat16*>(ep.gate_table);
  r.grow = gtab ? gtab + (int64_t)ep.gate_row * N : nullptr;
  r.gtrow = gtab ? static_cast<const __nv_bfloat16*>(ep.gate_t) + ((row_ok ? m / ep.rows_per_batch : 0) * 6 + ep.gate_row) * N
                 : nullptr;
  r.nbase = nbase;
  r.N = N;
  return r;
}

__device__ __forceinline__ void epi_fetch(const EpiRow& r, EpiStep& s, int c) {
  const int64_t n = r.nbase + 16 * c;
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int64_t nj = n + 8 * j;
    const bool in = nj < r.N;
    s.bias[j] = (r.bias && in) ? __ldg(reinterpret_cast<const uint4*>(r.bias + nj)) : make_uint4(0u, 0u, 0u, 0u);
    if (r.grow) {
      s.gtab[j] = in ? __ldg(reinterpret_cast<const uint4*>(r.grow + nj)) : make_uint4(0u, 0u, 0u, 0u);
      s.gt[j] = in ? __ldg(reinterpret_cast<const uint4*>(r.gtrow + nj)) : make_uint4(0u, 0u, 0u, 0u);
    }
  }
}

// ---- staged epilogue: shared-memory boxes + bulk-tensor copies --------------------------------
// An epilogue warp owns 32 accumulator rows (its TMEM lane quadrant) and NBOX boxes of 32 rows
// x 64 columns.  All of its global traffic is bulk-tensor copies through the box buffers in
// shared memory (rows of 128 bytes, 128-byte swizzle, so a lane reading or writing its own row
// hits no bank conflict): the residual box is loaded while the accumulator is still being
// computed, each lane adds its row in place, and the finished box is stored by one bulk copy,
// which also clips rows >= M and columns >= N.  Per-lane 16-byte loads and stores of 32
// different rows cost the SM sixteen times as many memory requests, which bounded the epilogue.
constexpr int EPI_BOX_COLS = 64;
constexpr int EPI_BOX_BYTES = 32 * EPI_BOX_COLS * 2;  // 4 KiB

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tmap, uint32_t smem_src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(tmap), "r"(smem_src), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all of this thread's bulk stores have finished READING shared memory (the staging boxes are free again)
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// generic-proxy writes to shared memory become visible to the async proxy (the bulk store)
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

struct EpiBox {
  uint32_t box_s;        // shared address of this warp's box 0
  unsigned char* row_g;  // generic address of this lane's 128-byte row of box 0
  uint32_t res_bar;      // mbarrier counting the residual loads of a tile
  uint32_t res_phase;
  uint32_t swz;          // lane & 7: the row's swizzle of its 16-byte pieces
};

// Start of a tile (before the accumulator is ready): once the previous tile's stores have read
// the boxes, the residual boxes of this tile are fetched into them.
template <int NBOX>
__device__ __forceinline__ void epi_box_begin(const EpiBox& eb, const EpiRow& row, bool use_res, int lane, int m_box,
                                              const CUtensorMap* tmRes) {
  if (lane == 0) bulk_wait_read_all();
  __syncwarp();
  if (use_res && lane == 0 && row.nbase < row.N) {
    int nb = 0;
#pragma unroll
    for (int j = 0; j < NBOX; ++j) nb += (row.nbase + EPI_BOX_COLS * j < row.N) ? 1 : 0;
    mbar_expect_tx(eb.res_bar, (uint32_t)(nb * EPI_BOX_BYTES));
#pragma unroll
    for (int j = 0; j < NBOX; ++j)
      if (row.nbase + EPI_BOX_COLS * j < row.N)
        tma_load_2d(eb.box_s + j * EPI_BOX_BYTES, tmRes, eb.res_bar, (int)(row.nbase + EPI_BOX_COLS * j), m_box);
  }
}

// The accumulator is complete: read it 16 columns at a time, apply the epilogue in the boxes and
// store them.  st[0] must hold the side operands of step 0 (epi_fetch).  Returns false when the
// wait for the residual was abandoned.
template <int NCHUNK, bool SCALE>
__device__ __forceinline__ bool epi_box_drain(EpiBox& eb, const EpiRow& row, const EpiParams& ep, uint32_t taddr,
                                              EpiStep (&st)[2], bool use_res, bool box_rows_in, int lane, int m_box,
                                              const CUtensorMap* tmOut, float alpha, volatile int* abort_flag,
                                              int* status_word) {
  const int64_t nbase = row.nbase, N = row.N;
  if (nbase < N) {
    tmem_ld_32x16(taddr, st[0].acc);
    if (use_res) {
      if (!mbar_wait(eb.res_bar, eb.res_phase, abort_flag, 5, status_word)) return false;
      eb.res_phase ^= 1u;
    }
  }
#pragma unroll
  for (int c = 0; c < NCHUNK; ++c) {
    const int64_t n = nbase + 16 * c;
    if (n >= N) break;  // uniform: the rest of this half lies outside the matrix
    constexpr int CPB = EPI_BOX_COLS / 16;  // 16-column steps per box
    const int j = c / CPB, cc = c % CPB;
    EpiStep& cur = st[c & 1];
    tmem_ld_wait();
    const bool more = (c + 1 < NCHUNK) && (n + 16 < N);
    if (more) {
      tmem_ld_32x16(taddr + (uint32_t)(16 * (c + 1)), st[(c + 1) & 1].acc);
      epi_fetch(row, st[(c + 1) & 1], c + 1);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (n + 8 * h < N) {
        float v[8], f[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(cur.acc[8 * h + e]);
        if (SCALE) {
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] *= alpha;
        }
        if (row.bias) {
          unpack8(cur.bias[h], f);
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] += f[e];
        }
        if (ep.act == 1) {
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = fast_silu(v[e]);
        } else if (ep.act == 2) {
#pragma unroll
          for (int e = 0; e < 8; ++e)
            if (n + 8 * h + e < ep.relu_cols) v[e] = fmaxf(v[e], 0.f);
        } else if (ep.act == 3) {
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = gelu_tanh(v[e]);
        }
        if (row.grow) {
          float g[8];
          unpack8(cur.gtab[h], g);
          unpack8(cur.gt[h], f);
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] *= (g[e] + f[e]);
        }
        // 16-byte piece (2*cc + h) of this lane's 128-byte row of box j, swizzled by the row
        uint4* slot = reinterpret_cast<uint4*>(eb.row_g + j * EPI_BOX_BYTES + ((((uint32_t)(2 * cc + h)) ^ eb.swz) << 4));
        if (use_res) {
          unpack8(*slot, f);
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] += f[e];
        }
        *slot = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
      }
    }
    if (cc == CPB - 1 || !more) {  // box j is complete
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0 && box_rows_in) {
        tma_store_2d(tmOut, eb.box_s + j * EPI_BOX_BYTES, (int)(nbase + EPI_BOX_COLS * j), m_box);
        bulk_commit();
      }
    }
  }
  return true;
}

// ---- the same epilogue on an accumulator that has been copied into registers first ---------------
// Where a kernel has one accumulator buffer only, the epilogue warps copy their part of it out of tensor
// memory in one go (NCHUNK back-to-back loads), hand the buffer back to the MMA issuer, and only then do the
// arithmetic and the stores - which then run under the next tile's MMAs.
template <int NCHUNK>
__device__ __forceinline__ void epi_acc_load(uint32_t taddr, uint32_t (&acc)[NCHUNK][16]) {
#pragma unroll
  for (int c = 0; c < NCHUNK; ++c) tmem_ld_32x16(taddr + (uint32_t)(16 * c), acc[c]);
  tmem_ld_wait();
}

struct EpiSide {
  uint4 bias[2], gtab[2], gt[2];
};
__device__ __forceinline__ void epi_fetch_side(const EpiRow& r, EpiSide& s, int c) {
  const int64_t n = r.nbase + 16 * c;
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int64_t nj = n + 8 * j;
    const bool in = nj < r.N;
    s.bias[j] = (r.bias && in) ? __ldg(reinterpret_cast<const uint4*>(r.bias + nj)) : make_uint4(0u, 0u, 0u, 0u);
    if (r.grow) {
      s.gtab[j] = in ? __ldg(reinterpret_cast<const uint4*>(r.grow + nj)) : make_uint4(0u, 0u, 0u, 0u);
      s.gt[j] = in ? __ldg(reinterpret_cast<const uint4*>(r.gtrow + nj)) : make_uint4(0u, 0u, 0u, 0u);
    }
  }
}

template <int NCHUNK, bool SCALE>
__device__ __forceinline__ bool epi_box_drain_regs(EpiBox& eb, const EpiRow& row, const EpiParams& ep,
                                                   const uint32_t (&acc)[NCHUNK][16], bool use_res, bool box_rows_in, int lane,
                                                   int m_box, const CUtensorMap* tmOut, float alpha, volatile int* abort_flag,
                                                   int* status_word) {
  const int64_t nbase = row.nbase, N = row.N;
  EpiSide side[2];
  if (nbase < N) {
    epi_fetch_side(row, side[0], 0);
    if (use_res) {
      if (!mbar_wait(eb.res_bar, eb.res_phase, abort_flag, 5, status_word)) return false;
      eb.res_phase ^= 1u;
    }
  }
#pragma unroll
  for (int c = 0; c < NCHUNK; ++c) {
    const int64_t n = nbase + 16 * c;
    if (n >= N) break;  // uniform: the rest of this half lies outside the matrix
    constexpr int CPB = EPI_BOX_COLS / 16;
    const int j = c / CPB, cc = c % CPB;
    const EpiSide& cur = side[c & 1];
    const bool more = (c + 1 < NCHUNK) && (n + 16 < N);
    if (more) epi_fetch_side(row, side[(c + 1) & 1], c + 1);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (n + 8 * h < N) {
        float v[8], f[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(acc[c][8 * h + e]);
        if (SCALE) {
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] *= alpha;
        }
        if (row.bias) {
          unpack8(cur.bias[h], f);
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] += f[e];
        }
        if (ep.act == 1) {
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = fast_silu(v[e]);
        } else if (ep.act == 2) {
#pragma unroll
          for (int e = 0; e < 8; ++e)
            if (n + 8 * h + e < ep.relu_cols) v[e] = fmaxf(v[e], 0.f);
        } else if (ep.act == 3) {
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = gelu_tanh(v[e]);
        }
        if (row.grow) {
          float g[8];
          unpack8(cur.gtab[h], g);
          unpack8(cur.gt[h], f);
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] *= (g[e] + f[e]);
        }
        uint4* slot = reinterpret_cast<uint4*>(eb.row_g + j * EPI_BOX_BYTES + ((((uint32_t)(2 * cc + h)) ^ eb.swz) << 4));
        if (use_res) {
          unpack8(*slot, f);
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] += f[e];
        }
        *slot = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
      }
    }
    if (cc == CPB - 1 || !more) {  // box j is complete
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0 && box_rows_in) {
        tma_store_2d(tmOut, eb.box_s + j * EPI_BOX_BYTES, (int)(nbase + EPI_BOX_COLS * j), m_box);
        bulk_commit();
      }
    }
  }
  return true;
}

// ---- CTA pairs (clusters of two, tcgen05 cta_group::2) ------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load whose completion bytes are counted on a barrier that may live in the peer CTA
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const CUtensorMap* tmap, uint32_t bar_cluster_addr,
                                                 int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_dst), "l"(tmap), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives (once all prior MMAs of this thread completed) on the barrier at this offset in both CTAs
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(mask)
               : "memory");
}

// Order of the output tiles.  Row-major order makes the tiles in flight at one time (one per CTA pair) span two
// tile rows and every tile column, i.e. the whole weight matrix passes through L2 once per wave (50 MB for the
// 11 200-wide projection).  Walking groups of PAIR_GROUP_M tile rows column by column keeps a wave on a few
// columns of W and PAIR_GROUP_M row tiles of A instead (about 20 MB), which is what the L2 can hold next to the
// streaming output.
constexpr int PAIR_GROUP_M = 8;
__device__ __forceinline__ void pair_tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int per_group = PAIR_GROUP_M * tiles_n;
  const int g = tile / per_group, within = tile - g * per_group;
  const int rows = min(PAIR_GROUP_M, tiles_m - g * PAIR_GROUP_M);
  tn = within / rows;
  tm = g * PAIR_GROUP_M + (within - tn * rows);
}

// ---- host helpers -----------------------------------------------------------------------------
// kernel choice set by sana_gemm_set_variant: 0 = per problem, 1 = single-CTA kernels, 2 = CTA-pair kernels
int gemm_variant();
// 2-D tiled tensor map over a row-major [rows, cols] matrix of `elem_bytes`-wide elements, row
// stride ld_bytes; box = box_rows x box_cols, 128-byte swizzle, out-of-range reads give zeros.
int make_tmap_2d(CUtensorMap* tm, CUtensorMapDataType dtype, int elem_bytes, const void* base, int64_t rows,
                 int64_t cols, int64_t ld_bytes, int box_rows, int box_cols);
// General tiled map of `rank` (<= 5) dimensions, innermost first; strides_bytes has rank-1 entries
// (dimensions 1 .. rank-1), each a multiple of 16; out-of-range reads give zeros.
int make_tmap_tiled(CUtensorMap* tm, CUtensorMapDataType dtype, int rank, const void* base, const uint64_t* dims,
                    const uint64_t* strides_bytes, const uint32_t* box, bool swizzle128);

}  // namespace sana
